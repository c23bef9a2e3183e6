"""Issue rate of the decode kernel's tensor-core instruction (tcgen05.mma kind::f8f6f4, M128 x N x K32, A from tensor
memory) on every multiprocessor, for the operand widths N and issuer arrangements the kernel could use.

    BITSTACK_B200_LIB=bitstack_b200/libbitstack_b200_tuning.so python -m bitstack_b200.mma_rate_probe

Needs the tuning build of the library (`python -m bitstack_b200.build --tuning`): the probe kernel is not part of the
product.  Prints ns per MMA per multiprocessor and what that means in packed sign bytes per second (one MMA consumes
128 x 32 signs = 512 packed bytes).
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from . import _lib


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--iters", type=int, default=2000)
    args = ap.parse_args()
    _lib.load()
    tun = C.CDLL(_lib.LIB_PATH)
    if not hasattr(tun, "bsb_tuning_mma_rate"):
        raise SystemExit("this is the product library; point BITSTACK_B200_LIB at libbitstack_b200_tuning.so")
    tun.bsb_tuning_mma_rate.argtypes = [C.c_int32] * 5 + [C.POINTER(C.c_float)]
    tun.bsb_tuning_mma_rate.restype = C.c_int
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    print("| N | MMAs per commit | issuers per CTA | CTAs per SM | ns per MMA per SM | packed sign TB/s (all SMs) |")
    print("|---|---|---|---|---|---|")
    cases = [(n, 8, 1, 1) for n in (16, 32, 64, 128, 256)]
    cases += [(32, 1, 1, 1), (32, 4, 1, 1), (32, 8, 2, 1), (32, 8, 1, 2), (32, 8, 2, 2), (64, 8, 2, 2)]
    for n, per_commit, issuers, ctas in cases:
        out = C.c_float(0)
        with torch.cuda.device(0):
            rc = tun.bsb_tuning_mma_rate(n, per_commit, args.iters, issuers, ctas, C.byref(out))
        if rc != 0:
            print(f"| {n} | {per_commit} | {issuers} | {ctas} | failed ({rc}) | |")
            continue
        tbs = 512.0 / out.value * sms / 1e3   # bytes per ns per SM x SMs = GB/s -> TB/s
        print(f"| {n} | {per_commit} | {issuers} | {ctas} | {out.value:.1f} | {tbs:.2f} |")
    _lib.check_device_status()


if __name__ == "__main__":
    main()
