"""Sign packing on the device: same convention and call shapes as the reference's
pack_sign / unpack_sign (bitstack/utils/pack_utils.py:5-26), CUDA tensors only."""
from __future__ import annotations

import torch

from . import _lib


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise ValueError(f"{what}: expected a CUDA tensor (this package has no CPU path)")


def pack_sign(w_sign: torch.Tensor) -> torch.Tensor:
    """int8 tensor of +1/-1 (any shape) -> uint8 [ceil(numel/8)], first sign in the MSB.
    Raises AssertionError on values other than +1/-1, like the reference."""
    _need_cuda(w_sign, "pack_sign")
    s = w_sign.to(torch.int8).contiguous().view(-1)
    n = s.numel()
    packed = torch.empty((n + 7) // 8, dtype=torch.uint8, device=s.device)
    bad = torch.zeros(1, dtype=torch.int32, device=s.device)
    with torch.cuda.device(s.device):
        _lib.check(_lib.load().bsb_pack_sign(s.data_ptr(), n, packed.data_ptr(), bad.data_ptr(), _stream(s)), "pack_sign")
    assert int(bad.item()) == 0, "pack_sign expects only +1 / -1"
    return packed


def unpack_sign(packed: torch.Tensor, original_shape) -> torch.Tensor:
    """uint8 packed bits -> int8 tensor of +1/-1 with `original_shape`."""
    _need_cuda(packed, "unpack_sign")
    if packed.dtype != torch.uint8:
        raise ValueError(f"Expected packed tensor of dtype torch.uint8, but got {packed.dtype}")
    shape = torch.Size(original_shape)
    n = shape.numel()
    p = packed.contiguous().view(-1)
    if p.numel() * 8 < n:
        raise ValueError(f"unpack_sign: {p.numel()} bytes cannot hold {n} signs")
    out = torch.empty(n, dtype=torch.int8, device=p.device)
    with torch.cuda.device(p.device):
        _lib.check(_lib.load().bsb_unpack_sign(p.data_ptr(), n, out.data_ptr(), _stream(p)), "unpack_sign")
    return out.view(shape)
