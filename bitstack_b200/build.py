"""Build libbitstack_b200.so in-tree with nvcc for sm_100a.

    python -m bitstack_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (see include/bitstack_b200.h); it does
not link against torch.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbitstack_b200.so")
# side build with -DBSB_TUNING: the same library plus timing-experiment modes and a fault-injection mode of the decode
# kernel (bsb_tuning_set_mode / bsb_tuning_set_trace); the tests of the give-up path load it, the product never does
TUNING_LIB = os.path.join(HERE, "libbitstack_b200_tuning.so")
SOURCES = ["capi.cu", "pack_kernels.cu", "general_kernels.cu", "rebuild_gemm.cu", "gemv_tc5.cu", "gemm_tc5.cu", "signgemm_tc5.cu", "signgemm_mma.cu", "decode_glue.cu", "peer_reduce.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "rowops.cuh"), os.path.join(os.path.dirname(HERE), "include", "bitstack_b200.h")]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA toolkit is required to build bitstack_b200")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=None, lib_path: str = LIB, objdir_name: str = "build") -> str:
    """`extra_flags` / `lib_path` / `objdir_name` build a tuning variant beside the product library."""
    nvcc = _nvcc()
    objdir = os.path.join(HERE, objdir_name)
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [path] + HEADERS):
            cmd = [nvcc, "-c", path, "-o", obj] + FLAGS + list(extra_flags or []) + (["-Xptxas", "-v"] if verbose else [])
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(lib_path, objs):
        cmd = [nvcc, "-shared", "-o", lib_path] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        subprocess.check_call(cmd)
    return lib_path


def build_tuning(force: bool = False, verbose: bool = False) -> str:
    return build(force=force, verbose=verbose, extra_flags=["-DBSB_TUNING"], lib_path=TUNING_LIB, objdir_name="build_tuning")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--tuning" in sys.argv:
        print(build_tuning(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
