"""The give-up path of the time-bounded waits, exercised without faulting or hanging the GPU.

Every wait inside the tcgen05 kernels has a time limit.  The tuning build of the library (compiled with
-DBSB_TUNING, never loaded by the product) has a mode in which the decode kernel's Z' loader never loads: the
barrier the MMA issuer waits on is a flag that nothing sets.  With the limit lowered to 20 ms every role runs out of
its wait, the kernel returns normally, and the host must then see (a) a sticky non-zero status word, (b) NaN in
every output of the call, (c) a context that is still usable: the next call, in normal mode, is correct.
The experiment runs in a child process so that the tuning library and its status word stay out of the other tests.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import ctypes as C, os, sys
import numpy as np, torch
sys.path.insert(0, os.environ["BSB_ROOT"])
from oracle import bitstack_oracle as orc
from bitstack_b200 import _lib, BitStackLinear
lib = _lib.load()
tuning = C.CDLL(_lib.LIB_PATH)
dev = torch.device("cuda:0")
m, n, nb = 640, 1024, 3
q, u, vt = orc.synthetic_layer(m, n, nb, seed=1)
mod = BitStackLinear(w_bit=nb, in_features=n, out_features=m, k=16, bias=False, no_avd=False, dev=dev, fused_level=10)
for j in range(nb):
    getattr(mod, f"qweight_{j}").copy_(torch.from_numpy(q[j]))
    getattr(mod, f"u_{j}").copy_(torch.from_numpy(u[j]))
    getattr(mod, f"vt_{j}").copy_(torch.from_numpy(vt[j]))
mod.stack_blocks()
x_np = orc.synthetic_input(2, n, seed=2)
x = torch.from_numpy(x_np).to(dev)
good = mod(x)
torch.cuda.synchronize()
assert lib.bsb_set_wait_limit_ms(20) == 0
assert tuning.bsb_tuning_set_mode(3) == 0          # the Z' loader never loads
bad = mod(x)
code = C.c_int32(0)
rc = lib.bsb_read_status(C.byref(code), 0)
assert rc == -5 and code.value != 0, (rc, code.value)
assert bool(torch.isnan(bad).all()), "outputs of a timed-out call must be NaN"
assert tuning.bsb_tuning_set_mode(0) == 0
again = mod(x)                                      # the status is sticky: a later, healthy call does not clear it
rc = lib.bsb_read_status(C.byref(code), 1)
assert rc == -5 and code.value != 0
assert lib.bsb_read_status(C.byref(code), 1) == 0 and code.value == 0
assert torch.equal(again, good), "the context must stay usable after a give-up"
try:
    _lib.check_device_status()
except Exception as e:
    raise AssertionError(f"status should be clear now: {e}")
print("GIVE_UP_OK", flush=True)
'''


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_marks_outputs_nan():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from bitstack_b200 import build
    lib = build.TUNING_LIB
    if not os.path.exists(lib):
        lib = build.build_tuning()
    env = dict(os.environ, BITSTACK_B200_LIB=lib, BSB_ROOT=ROOT)
    out = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "GIVE_UP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]


def test_tuning_build_has_the_extra_entry_points_and_the_product_does_not():
    import ctypes
    from bitstack_b200 import _lib, build
    build.build()
    build.build_tuning()
    prod, tun = ctypes.CDLL(_lib.LIB_PATH), ctypes.CDLL(build.TUNING_LIB)
    assert hasattr(tun, "bsb_tuning_set_mode") and hasattr(tun, "bsb_tuning_set_trace")
    assert not hasattr(prod, "bsb_tuning_set_mode") and not hasattr(prod, "bsb_tuning_set_trace")
