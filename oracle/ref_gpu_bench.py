"""Time the reference's OWN fused levels (its Triton kernels, staged unchanged by oracle/make_ref.py) on this GPU next
to this library, on the same tensors.

    python oracle/ref_gpu_bench.py [--shapes 4096x4096,14336x4096] [--blocks 8] [--rows 1,16,2048] [--levels 2,3,5]

Per (shape, rows): median CUDA-event time of reference level 2 (unpack kernel + fused reconstruct kernel + F.linear),
level 3 (fused unpack-and-reconstruct kernel + F.linear) and level 5 (per-token reconstruct-and-forward; decode only,
3-D input) after an untimed warm-up call that lets Triton autotune, against `BitStackLinear` of this library at its
automatic level, with the L2 flushed between calls.  GB/s are algorithmic bytes
(blocks * (out*in/8 + 32*(out+in)) + 2*rows*(in+out)) over time.  Test / baseline infrastructure: imports the staged
reference, never imported by the package.
"""
import argparse
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from oracle.make_ref import import_reference  # noqa: E402


def timed(fn, flush, calls):
    out = []
    for _ in range(calls):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        out.append(s.elapsed_time(e) * 1e3)
    return float(np.median(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="4096x4096,14336x4096")
    ap.add_argument("--blocks", type=int, default=8)
    ap.add_argument("--rows", default="1,16,2048")
    ap.add_argument("--levels", default="2,3,5")
    ap.add_argument("--calls", type=int, default=5)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    from bitstack_b200 import BitStackLinear
    Ref = import_reference()
    dev = torch.device("cuda:0")
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    levels = [int(v) for v in a.levels.split(",")]
    print("| shape | blocks | rows | ours us (GB/s) | " + " | ".join(f"ref L{l} us (GB/s)" for l in levels) + " |")
    print("|---|---|---|---|" + "---|" * len(levels))
    for shp in a.shapes.split(","):
        m, n = (int(v) for v in shp.split("x"))
        nb = a.blocks
        g = torch.Generator(device=dev).manual_seed(m + n)
        q = torch.randint(0, 256, (nb, m * n // 8), dtype=torch.uint8, device=dev, generator=g)
        u = (torch.randn(nb, m, 16, device=dev, generator=g) * 0.05).abs().half()
        vt = (torch.randn(nb, 16, n, device=dev, generator=g) * 0.05).abs().half()
        ours = BitStackLinear(w_bit=0, in_features=n, out_features=m, k=16, bias=False, no_avd=False, dev=dev, fused_level=6)
        ours.qweight, ours.u, ours.vt, ours.w_bit, ours._stacked_blocks = q, u, vt, nb, nb
        refs = {}
        for l in levels:
            r = Ref(w_bit=nb, in_features=n, out_features=m, k=16, bias=False, no_avd=False, dev=dev, fused_level=l)
            for j in range(nb):
                setattr(r, f"qweight_{j}", q[j].clone())
                setattr(r, f"u_{j}", u[j].clone())
                setattr(r, f"vt_{j}", vt[j].clone())
            r.stack_blocks()
            refs[l] = r
        for rows in (int(v) for v in a.rows.split(",")):
            x = torch.randn(rows, n, device=dev, generator=g).half()
            byts = nb * (m * n // 8 + 32 * (m + n)) + 2 * rows * (m + n)
            y = ours(x)
            t_ours = timed(lambda: ours(x), flush, a.calls)
            cells = []
            for l in levels:
                if l == 5 and rows > 16:
                    cells.append("- (per-token kernel)")
                    continue
                xin = x.view(1, rows, n) if l == 5 else x
                try:
                    t0 = time.perf_counter()
                    yr = refs[l](xin)                      # warm-up: Triton autotune happens here
                    torch.cuda.synchronize()
                    tune = time.perf_counter() - t0
                    err = float((yr.reshape(rows, m).float() - y.float()).abs().max() / y.float().abs().max())
                    t = timed(lambda: refs[l](xin), flush, a.calls)
                    cells.append(f"{t:.1f} ({byts / t / 1e3:.0f}); diff {err:.1e}; tune {tune:.0f}s")
                except Exception as e:  # noqa: BLE001
                    cells.append(f"failed: {type(e).__name__}: {str(e)[:60]}")
            print(f"| {m}x{n} | {nb} | {rows} | {t_ours:.1f} ({byts / t_ours / 1e3:.0f}) | " + " | ".join(cells) + " |", flush=True)


if __name__ == "__main__":
    main()
