"""No-GPU checks of the C-ABI library: it builds/loads and exports every symbol the
public header declares, and the ctypes signatures cover exactly that set."""
import ctypes
import os
import re

import pytest

from bitstack_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    if not os.path.exists(_lib.LIB_PATH):
        from bitstack_b200.build import build
        build()
    return ctypes.CDLL(_lib.LIB_PATH)


def _header_functions():
    text = open(os.path.join(ROOT, "include", "bitstack_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built_lib):
    names = _header_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(built_lib, n), f"{n} declared in the header but not exported"


def test_ctypes_signatures_match_header():
    assert sorted(_lib.SIGNATURES) == _header_functions()


def test_struct_layout_matches_header():
    # 5 pointers + 3 int64 + 4 int32 on a 64-bit ABI
    assert ctypes.sizeof(_lib.BsbWeight) == 5 * 8 + 3 * 8 + 4 * 4
    assert _lib.BsbWeight.blocks.offset == 76


def test_version_and_error_string_without_gpu(built_lib):
    lib = _lib.load()
    assert lib.bsb_version() >= 100
    assert isinstance(lib.bsb_last_error(), bytes)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.BitStackLibraryError):
        _lib.load()


def test_module_rejects_cpu_inputs():
    import torch
    from bitstack_b200 import BitStackLinear, pack_sign
    m = BitStackLinear(w_bit=2, in_features=128, out_features=16, k=16, bias=False, no_avd=False, dev="cpu")
    with pytest.raises(ValueError):
        m(torch.zeros(1, 128, dtype=torch.float16))
    with pytest.raises(ValueError):
        pack_sign(torch.ones(8, dtype=torch.int8))
    m.fused_level = 42
    with pytest.raises(ValueError, match="Invalid fused_level"):
        m(torch.zeros(1, 128, dtype=torch.float16))
    with pytest.raises(NotImplementedError):
        BitStackLinear(w_bit=1, in_features=8, out_features=8, k=1, bias=False, no_avd=True, dev="cpu")


def test_module_mirrors_reference_buffers():
    import torch
    from bitstack_b200 import BitStackLinear
    lin = torch.nn.Linear(96, 64, bias=True)
    m = BitStackLinear.from_linear(lin, w_bit=3, k=16, bias=True, name="layer.0.self_attn.q_proj", init_only=True)
    sd = m.state_dict()
    assert sorted(sd) == sorted([f"{p}_{i}" for p in ("qweight", "u", "vt") for i in range(3)] + ["bias"])
    assert sd["qweight_0"].shape == (64 * 96 // 8,) and sd["qweight_0"].dtype == torch.uint8
    assert sd["u_2"].shape == (64, 16) and sd["u_2"].dtype == torch.float16
    assert sd["vt_1"].shape == (16, 96) and sd["vt_1"].dtype == torch.float16
    assert m.memory_per_bit() == 64 * 96 // 8 + 2 * 16 * (64 + 96)
    m.pop_one_bit(); assert m.w_bit == 2
    m.add_one_bit(); assert m.w_bit == 3
    m.set_bit(1); assert m.w_bit == 1
    m.set_bit(3)
    m.stack_blocks()
    assert m.qweight.shape == (3, 768) and m.u.shape == (3, 64, 16) and m.vt.shape == (3, 16, 96)
    assert "qweight_0" not in m.state_dict()
