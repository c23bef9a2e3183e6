"""Time the forward of ONE BitStack projection on synthetic weights.

    python -m bitstack_b200.layer_bench --out 14336 --in 4096 --blocks 16 --rows 1 --calls 10

Prints, per call path, the median device time of the main kernel (CUDA events recorded by the
library around its own launch, on the launching stream) and of the whole call, with the
algorithmic bytes `blocks*(out*in/8 + 32*(out+in)) + 2*rows*(in+out)` over that time.  The L2 is
flushed (a 512 MB fill) between timed calls.  It is also the small, single-kernel command
that profiler captures of the decode kernel are taken with (`--calls 1 --no-flush`).

Weights: uniform random sign bytes, |N(0, 0.05)| factors (the value distribution of the absolute-value
decomposition, bitstack/modules/BitStackLinear.py:49-75), N(0, 1) activations.
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np
import torch

from . import _lib
from .linear import BitStackLinear


def synthetic_projection(out_features: int, in_features: int, blocks: int, level: int, dev, seed: int = 0) -> BitStackLinear:
    mod = BitStackLinear(w_bit=0, in_features=in_features, out_features=out_features, k=16, bias=False,
                         no_avd=False, dev=dev, fused_level=level)
    g = torch.Generator(device=dev).manual_seed(seed + out_features + in_features)
    mod.qweight = torch.randint(0, 256, (blocks, out_features * in_features // 8), dtype=torch.uint8, device=dev, generator=g)
    mod.u = (torch.randn(blocks, out_features, 16, device=dev, generator=g) * 0.05).abs().half()
    mod.vt = (torch.randn(blocks, 16, in_features, device=dev, generator=g) * 0.05).abs().half()
    mod.w_bit = blocks
    mod._stacked_blocks = blocks
    return mod


def algorithmic_bytes(out_features: int, in_features: int, blocks: int, rows: int) -> int:
    return blocks * (out_features * in_features // 8 + 32 * (out_features + in_features)) + 2 * rows * (in_features + out_features)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", type=int, default=14336)
    ap.add_argument("--in", dest="inp", type=int, default=4096)
    ap.add_argument("--blocks", type=int, default=16)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--level", type=int, default=10, help="fused_level of BitStackLinear (10 = tcgen05 decode kernel)")
    ap.add_argument("--calls", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--graph", type=int, default=0, help="also time N back-to-back calls replayed as one CUDA graph")
    ap.add_argument("--pdl", action="store_true", help="launch the decode kernel as a programmatic dependent of the Z' kernel")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("layer_bench needs a CUDA device")
    dev = torch.device("cuda:0")
    lib = _lib.load()
    lib.bsb_set_dependent_launch(1 if a.pdl else 0)
    mod = synthetic_projection(a.out, a.inp, a.blocks, a.level, dev)
    x = torch.randn(a.rows, a.inp, device=dev).half()
    flush = None if a.no_flush else torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    for _ in range(a.warmup):
        mod(x)
    torch.cuda.synchronize()
    cap = 4 * max(a.calls, 1) * max(a.rows, 1)
    lib.bsb_debug_profile_start(min(cap, 4096))
    whole = []
    for _ in range(a.calls):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        mod(x)
        e.record()
        torch.cuda.synchronize()
        whole.append(s.elapsed_time(e) * 1e3)
    buf = (C.c_float * 4096)()
    k = C.c_int32(0)
    lib.bsb_debug_profile_stop(buf, 4096, C.byref(k))
    main_us = np.array(buf[: k.value]) * 1e3
    b = algorithmic_bytes(a.out, a.inp, a.blocks, a.rows)
    line = f"{a.out}x{a.inp} blocks={a.blocks} rows={a.rows} level={a.level}: whole call median {np.median(whole):.1f} us ({b / np.median(whole) / 1e3:.1f} GB/s)"
    if k.value:
        line += f"; main kernel median {np.median(main_us):.1f} us ({b / np.median(main_us) / 1e3:.1f} GB/s) over {k.value} launches"
        if a.rows > 4 and a.level in (0, 9):
            fl = 2.0 * a.rows * a.out * a.inp
            line += f" = {fl / np.median(main_us) / 1e6:.1f} TFLOP/s for the GEMM alone"
    print(line)
    if a.graph > 0:
        # steady-state cost of a call inside a captured decode step: launch gaps included, caches warm
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            mod(x)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for _ in range(a.graph):
                    mod(x)
            g.replay()
            st.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(st)
            for _ in range(5):
                g.replay()
            e.record(st)
            st.synchronize()
        per = s.elapsed_time(e) * 1e3 / (5 * a.graph)
        print(f"  graph replay of {a.graph} calls: {per:.1f} us per call ({b / per / 1e3:.1f} GB/s; L2-warm if the weight fits)")


if __name__ == "__main__":
    main()
