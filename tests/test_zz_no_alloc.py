"""The allocation-free forward (`bsb_linear_forward_noalloc`) against the regular entry point.

This file is named so that pytest collects it last: a run that stops at the first failure
has then already executed every other test.

Who needs the entry point: hosts that give a plug-in a fixed set of device buffers and allow
no allocation afterwards (a server with a frozen memory plan, a framework whose pool owns the
GPU), and therefore cannot lend a workspace either.  The library keeps a 16 MiB scratch area
inside its own image for them.  The test calls the entry point through the C ABI twice in a
row -- the area is shared between calls and keeps the previous call's contents -- and
compares with `bsb_linear_forward`, which runs the same kernel on a caller-provided
workspace: results must agree to fp16 rounding (they are in fact identical).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import bitstack_oracle as orc

pytestmark = pytest.mark.gpu


def _module(m, n, nb, seed, dev):
    from bitstack_b200 import BitStackLinear
    q, u, vt = orc.synthetic_layer(m, n, nb, seed)
    mod = BitStackLinear(w_bit=nb, in_features=n, out_features=m, k=16, bias=False, no_avd=False, dev=dev, fused_level=10)
    for j in range(nb):
        getattr(mod, f"qweight_{j}").copy_(torch.from_numpy(q[j]))
        getattr(mod, f"u_{j}").copy_(torch.from_numpy(u[j]))
        getattr(mod, f"vt_{j}").copy_(torch.from_numpy(vt[j]))
    mod.stack_blocks()
    return mod, (q, u, vt)


def test_noalloc_forward_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from bitstack_b200 import _lib
    dev = torch.device("cuda:0")
    lib = _lib.load()
    assert lib.bsb_noalloc_scratch_bytes() == 16 << 20
    stream = torch.cuda.current_stream(dev).cuda_stream
    # two different layers back to back: the second call finds the first call's scratch contents
    for (m, n, nb, rows, seed) in ((1024, 4096, 7, 1, 5), (512, 1792, 3, 2, 6)):
        mod, (q, u, vt) = _module(m, n, nb, seed, dev)
        x_np = orc.synthetic_input(rows, n, seed + 100)
        x = torch.from_numpy(x_np).to(dev)
        ref = mod(x)                                   # bsb_linear_forward, caller workspace
        d = mod.weight_desc(dev)
        # once with the caller's precomputed max |vt|, once without it: the entry point then computes it into a
        # corner of its built-in area
        for absmax in (d.vt_absmax, None):
            d2 = _lib.BsbWeight()
            C.memmove(C.byref(d2), C.byref(d), C.sizeof(_lib.BsbWeight))
            d2.vt_absmax = absmax
            y = torch.full((rows, m), float("nan"), dtype=torch.float16, device=dev)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(dev)[0]      # the driver's own count: sees any cudaMalloc in the process
            before = torch.cuda.memory_allocated(dev)
            rc = lib.bsb_linear_forward_noalloc(C.byref(d2), x.data_ptr(), rows, n, y.data_ptr(), m, stream)
            assert rc == 0, lib.bsb_last_error()
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated(dev) == before
            assert torch.cuda.mem_get_info(dev)[0] >= free_before
            err = (y.float() - ref.float()).abs().max().item()
            assert err <= 2e-3 * ref.float().abs().max().item(), (m, n, nb, err)
            y64 = orc.forward_f64(x_np, q, u, vt, nb)
            assert orc.max_normalised_error(y.float().cpu().numpy(), y64) <= 4e-3


def test_noalloc_rejects_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from bitstack_b200 import BitStackLinear, _lib
    dev = torch.device("cuda:0")
    lib = _lib.load()
    # 40 blocks x 16384 input features need more than the 16 MiB built-in area
    nb, m, n = 40, 128, 16384
    mod = BitStackLinear(w_bit=0, in_features=n, out_features=m, k=16, bias=False, no_avd=False, dev=dev, fused_level=10)
    mod.qweight = torch.zeros(nb, m * n // 8, dtype=torch.uint8, device=dev)
    mod.u = torch.zeros(nb, m, 16, dtype=torch.float16, device=dev)
    mod.vt = torch.zeros(nb, 16, n, dtype=torch.float16, device=dev)
    mod.w_bit = nb
    mod._stacked_blocks = nb
    d = mod.weight_desc(dev)
    x = torch.zeros(1, n, dtype=torch.float16, device=dev)
    y = torch.zeros(1, m, dtype=torch.float16, device=dev)
    rc = lib.bsb_linear_forward_noalloc(C.byref(d), x.data_ptr(), 1, n, y.data_ptr(), m, None)
    assert rc == -4 and b"scratch" in lib.bsb_last_error()
    # a shape the decode kernel does not take is an argument error, not a fault
    mod2, _ = _module(64, 128, 1, 3, dev)
    d2 = mod2.weight_desc(dev)
    d2.in_features = 96
    rc = lib.bsb_linear_forward_noalloc(C.byref(d2), x.data_ptr(), 1, 96, y.data_ptr(), 64, None)
    assert rc == -1
    # no input features at all, and a block stride shorter than a block: rejected on the host like everywhere else
    d3 = mod2.weight_desc(dev)
    d3.in_features = 0
    assert lib.bsb_linear_forward_noalloc(C.byref(d3), x.data_ptr(), 1, 128, y.data_ptr(), 64, None) == -1
    mod3, _ = _module(64, 128, 2, 4, dev)
    d4 = mod3.weight_desc(dev)
    d4.q_block_stride = 16
    assert lib.bsb_linear_forward_noalloc(C.byref(d4), x.data_ptr(), 1, 128, y.data_ptr(), 64, None) == -1
    assert b"q_block_stride" in lib.bsb_last_error()
