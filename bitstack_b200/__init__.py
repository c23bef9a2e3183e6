"""bitstack_b200: the BitStack residual-block linear layer on B200 (sm_100a).

Public surface (mirrors the reference's operator API):
    BitStackLinear            module with the reference's constructor / buffers / methods
    pack_sign, unpack_sign    sign bit packing on the device
    forward_grouped           several projections of one input in one launch sequence
    loader                    budget selection (compression_config.json) and partial safetensors loading
    importance                block-importance scoring loop (reduced_ppl_average.json) and the order it implies
"""
from .linear import BitStackLinear, forward_grouped, get_workspace
from .pack import pack_sign, unpack_sign
from . import loader
from . import importance

__all__ = ["BitStackLinear", "forward_grouped", "get_workspace", "pack_sign", "unpack_sign", "loader", "importance"]
