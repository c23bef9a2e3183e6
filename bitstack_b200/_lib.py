"""ctypes binding of libbitstack_b200.so (the C ABI in include/bitstack_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails the
caller gets an exception.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BITSTACK_B200_LIB") or os.path.join(_HERE, "libbitstack_b200.so")

ALGO_AUTO, ALGO_GENERAL, ALGO_REBUILD_GEMM, ALGO_GEMV_TC5, ALGO_SIGN_GEMM, ALGO_SIGN_GEMM_MMA = 0, 1, 3, 4, 5, 6


class BsbWeight(C.Structure):
    """Mirror of `struct bsb_weight`."""
    _fields_ = [
        ("qweight", C.c_void_p), ("u", C.c_void_p), ("vt", C.c_void_p), ("bias", C.c_void_p),
        ("vt_absmax", C.c_void_p),
        ("q_block_stride", C.c_int64), ("u_block_stride", C.c_int64), ("vt_block_stride", C.c_int64),
        ("out_features", C.c_int32), ("in_features", C.c_int32), ("k", C.c_int32), ("blocks", C.c_int32),
    ]


class BitStackLibraryError(RuntimeError):
    pass


_lib = None

# every symbol include/bitstack_b200.h declares: (restype, argtypes)
_P, _I64, _I32 = C.c_void_p, C.c_int64, C.c_int32
_WP = C.POINTER(BsbWeight)
SIGNATURES = {
    "bsb_version": (C.c_int, []),
    "bsb_last_error": (C.c_char_p, []),
    "bsb_device_info": (C.c_int, [C.POINTER(C.c_int)] * 3),
    "bsb_pack_sign": (C.c_int, [_P, _I64, _P, _P, _P]),
    "bsb_unpack_sign": (C.c_int, [_P, _I64, _P, _P]),
    "bsb_reconstruct_weight": (C.c_int, [_WP, _P, _P]),
    "bsb_vt_absmax": (C.c_int, [_WP, _P, _P]),
    "bsb_linear_workspace_bytes": (_I64, [_WP, _I64, C.c_int]),
    "bsb_linear_forward": (C.c_int, [_WP, _P, _I64, _I64, _P, _I64, _P, _I64, C.c_int, _P]),
    "bsb_linear_forward_partial": (C.c_int, [_WP, _P, _I64, _I64, _P, _I64, _P, _I64, C.c_int, _P]),
    "bsb_linear_forward_grouped": (C.c_int, [_WP, _I32, _P, _I64, _I64, C.POINTER(_P), C.POINTER(_I64), _P, _I64, C.c_int, _P]),
    "bsb_linear_forward_grouped_ex": (C.c_int, [_WP, _I32, _P, _I64, _I64, _P, C.POINTER(_P), C.POINTER(_I64), _P, _I64, _P]),
    "bsb_linear_grouped_workspace_bytes": (_I64, [_WP, _I32, _I64, C.c_int]),
    "bsb_add_rmsnorm": (C.c_int, [_P, _P, _P, C.c_float, _P, _P, _I64, _I32, _P]),
    "bsb_rope_cache": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _P]),
    "bsb_decode_attention": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _P, _I64, _P]),
    "bsb_decode_attention_scratch_bytes": (C.c_int64, [_I32, _I32, _I32]),
    "bsb_greedy_step": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P]),
    "bsb_silu_mul": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _P]),
    "bsb_peer_area_bytes": (_I64, [_I32, _I32, _I32]),
    "bsb_peer_alloc": (C.c_int, [_I64, C.POINTER(_P), _P]),
    "bsb_peer_open": (C.c_int, [_P, C.POINTER(_P)]),
    "bsb_peer_close": (C.c_int, [_P, _I32]),
    "bsb_peer_allreduce_add_rmsnorm": (C.c_int, [C.POINTER(_P), _I32, _I32, _I32, _I32, _P, _I64, _I32, _I32, _P, _P, C.c_float, _P, _P, _P]),
    "bsb_noalloc_scratch_bytes": (_I64, []),
    "bsb_linear_forward_noalloc": (C.c_int, [_WP, _P, _I64, _I64, _P, _I64, _P]),
    "bsb_read_status": (C.c_int, [C.POINTER(C.c_int32), _I32]),
    "bsb_set_wait_limit_ms": (C.c_int, [_I32]),
    "bsb_set_dependent_launch": (C.c_int, [_I32]),
    "bsb_debug_launch_count": (_I64, []),
    "bsb_debug_profile_start": (C.c_int, [_I32]),
    "bsb_debug_profile_stop": (C.c_int, [C.POINTER(C.c_float), _I32, C.POINTER(_I32)]),
    "bsb_linear_forward_host": (C.c_int, [_WP, _P, _I64, _P, _P, _P, _P, _I64, C.c_int, _P]),
}


def load():
    """Load the library once; raises BitStackLibraryError when it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BitStackLibraryError(
            f"{LIB_PATH} not found: build it with `python -m bitstack_b200.build` "
            "(there is no CPU fallback for the BitStack kernels)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class BitStackDeviceTimeout(BitStackLibraryError):
    """A time-bounded wait inside a kernel gave up; the outputs of that call are NaN."""


def check(rc: int, what: str):
    if rc != 0:
        msg = load().bsb_last_error().decode(errors="replace")
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        if rc == -5:
            raise BitStackDeviceTimeout(f"{what}: {msg}")
        raise BitStackLibraryError(f"{what} failed ({rc}): {msg}")


def check_device_status(clear: bool = True) -> None:
    """Synchronises the current device and raises BitStackDeviceTimeout if any kernel of the library gave up a wait
    since the status was last cleared.  Call it wherever the host waits for results anyway."""
    code = C.c_int32(0)
    check(load().bsb_read_status(C.byref(code), 1 if clear else 0), "device status")
