"""Wall-clock timeline of the projection calls inside a graph-replayed decode step.

    BITSTACK_B200_LIB=bitstack_b200/libbitstack_b200_tuning.so python -m bitstack_b200.step_timeline [--layers 6]

Needs the tuning build of the library (`python -m bitstack_b200.build --tuning`), whose decode kernels write
`globaltimer` marks into a buffer registered with `bsb_tuning_set_timeline`: per call, when its operand-preparation
CTAs entered / were released / finished, when the decode CTAs entered, consumed their first operand slab and left.
A few layers of the 8B architecture with the benchmark's seeded block counts are built, one decode step is captured
as a CUDA graph, replayed, and the marks of one replay are printed in microseconds from the step's first mark, with
the time each call was busy and the gap to the next call.
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np
import torch

from . import _lib, decode

MARKS = ["z_in", "z_go", "z_end", "g_in", "g_z1", "g_epi", "g_end", "z_max", "g_inL", "z_inL", "g_out1", "g_z1L"]
GROUPS = [("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("self_attn.o_proj",),
          ("mlp.gate_proj", "mlp.up_proj"), ("mlp.down_proj",)]


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--layers", type=int, default=6)
    a = ap.parse_args()
    lib = _lib.load()
    tun = C.CDLL(_lib.LIB_PATH)
    if not hasattr(tun, "bsb_tuning_set_timeline"):
        raise SystemExit("this needs the tuning build: set BITSTACK_B200_LIB to libbitstack_b200_tuning.so")
    dev = torch.device("cuda:0")
    L = a.layers
    shape = decode.LlamaShape("8b-slice", L, 4096, 32, 8, 14336)
    counts = decode.seeded_block_counts(shape, seed=1234, lo=2, hi=16, target_bytes=int(5.5e9) * L // 32)
    m = decode.BitStackLlamaDecoder(shape, counts, dev, seed=7, max_len=768, batch=1)
    m.prefill(torch.randint(0, shape.vocab, (1, 512), device=dev))
    st = torch.cuda.Stream(dev)
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        for _ in range(2):
            m.decode_step()
    ncall, nm = 4 * L, len(MARKS)
    buf = torch.zeros(ncall * nm, dtype=torch.int64, device=dev)
    tun.bsb_tuning_set_timeline(C.c_void_p(buf.data_ptr()), ncall)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        m.decode_step()
    tun.bsb_tuning_set_timeline(None, 0)
    init = torch.zeros(ncall, nm, dtype=torch.int64)
    init[:, [0, 1, 3, 4, 10]] = -1          # "first ..." marks are minima
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    buf.copy_(init.view(-1))
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    t = buf.cpu().numpy().astype(np.uint64).reshape(ncall, nm)
    t0 = int(t[0, 0])
    shapes = shape.proj_shapes()
    print("call: " + " ".join(f"{n:>7}" for n in MARKS) + "   | busy  gap to next   MB")
    tot_busy = tot_gap = 0.0
    for i in range(ncall):
        r = [(int(v) - t0) / 1e3 for v in t[i]]
        lay, gi = divmod(i, 4)
        mb = sum(counts[f"layer.{lay}.{p}"] * decode.block_bytes(*shapes[p]) for p in GROUPS[gi]) / 1e6
        busy = r[6] - r[4]
        gap = ((int(t[i + 1, 4]) - t0) / 1e3 - r[6]) if i + 1 < ncall else float("nan")
        tot_busy += busy
        if i + 1 < ncall:
            tot_gap += gap
        print(f"{i:4d}: " + " ".join(f"{v:7.1f}" for v in r) + f"   | {busy:5.1f}  {gap:5.1f}   {mb:6.1f}")
    print(f"sum busy (first slab consumed -> last CTA out) {tot_busy:.1f} us, sum of gaps {tot_gap:.1f} us over {ncall} calls")
    lib.bsb_read_status(C.byref(C.c_int32(0)), 0)


if __name__ == "__main__":
    main()
