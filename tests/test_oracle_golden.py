"""The CPU oracle against fixtures produced by running the reference itself
(tests/golden/make_golden.py).  No GPU, no reference checkout needed."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import bitstack_oracle as orc


def test_pack_known_answer(golden_dir):
    z = np.load(os.path.join(golden_dir, "pack_kat.npz"))
    assert z["kat_packed"].tolist() == [128, 1]
    assert orc.pack_sign(z["kat_sign"]).tolist() == [128, 1]
    assert np.array_equal(orc.unpack_sign(np.array([128, 1], np.uint8), (16,)), z["kat_sign"])


def test_pack_unpack_match_reference_bytes(golden_dir):
    z = np.load(os.path.join(golden_dir, "pack_kat.npz"))
    for i in range(int(z["n_cases"])):
        s, p = z[f"sign_{i}"], z[f"packed_{i}"]
        assert np.array_equal(orc.pack_sign(s), p), f"case {i} shape {s.shape}"
        assert np.array_equal(orc.unpack_sign(p, s.shape), s)
        assert torch.equal(orc.unpack_sign_t(p, s.shape), torch.from_numpy(s))


def test_pack_rejects_non_sign():
    with pytest.raises(AssertionError):
        orc.pack_sign(np.array([1, 0, -1], dtype=np.int8))


@pytest.mark.parametrize("fname", ["decomp_small.npz", "decomp_1024.npz"])
def test_forward_l0_bit_identical_to_reference(golden_dir, fname):
    z = np.load(os.path.join(golden_dir, fname))
    bias = z["bias"] if "bias" in z.files else None
    for rows in z["rows"]:
        x = z[f"x_{rows}"]
        for b in z["bits"]:
            y_ref = z[f"y_{rows}_{b}"]
            y = orc.forward_l0(x, z["qweight"], z["u"], z["vt"], int(b), bias).numpy()
            # same primitive ops on the same library: expect identical fp16 results,
            # allow one fp16 ulp of the output scale for a different thread count
            assert orc.max_normalised_error(y, y_ref) <= 2e-3
            # and the fp64 meaning of the stored data agrees within the oracle's noise floor
            y64 = orc.forward_f64(x, z["qweight"], z["u"], z["vt"], int(b), bias)
            assert orc.max_normalised_error(y64, y_ref) <= 5e-3
            assert orc.rel_l2_error(y64, y_ref) <= 5e-3


def test_decomposition_restatement_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "decomp_small.npz"))
    q, u, vt = orc.decompose_weight(z["weight"], niter=4, k=16)
    # sign matrices: identical except where the residual is within rounding of zero
    frac = np.mean(np.unpackbits(q.numpy() ^ z["qweight"]))
    assert frac < 1e-3
    # first block does not depend on any earlier rounding: must match exactly in sign
    assert np.array_equal(q[0].numpy(), z["qweight"][0])
    w_ref = orc.reconstruct_f64(z["qweight"], z["u"], z["vt"], 4, 64, 96)
    w_new = orc.reconstruct_f64(q.numpy(), u.numpy(), vt.numpy(), 4, 64, 96)
    assert orc.max_normalised_error(w_new, w_ref) < 1e-3
    # and the decomposition really approximates the weight it came from
    assert orc.rel_l2_error(w_ref, z["weight"]) < 0.2


def test_synthetic_l0_outputs(golden_dir):
    z = np.load(os.path.join(golden_dir, "synth_l0.npz"))
    for (m, n, nb, seed, rows, a) in z["cases"]:
        q, u, vt = orc.synthetic_layer(int(m), int(n), int(nb), int(seed))
        x = orc.synthetic_input(int(rows), int(n), int(seed) + 1000)
        y_ref = z[f"y_{m}_{n}_{seed}_{rows}_{a}"]
        y = orc.forward_l0(x, q, u, vt, int(a)).numpy()
        assert orc.max_normalised_error(y, y_ref) <= 2e-3
        y64 = orc.forward_f64(x, q, u, vt, int(a))
        assert orc.max_normalised_error(y64, y_ref) <= 5e-3


def test_budget_lookup_and_config_generation(golden_dir):
    g = json.load(open(os.path.join(golden_dir, "budget.json")))
    cfgs = orc.generate_configs(g["order"], g["memory_per_bit"], g["total"])
    assert cfgs == g["configs"]
    for mb, layers in g["picks"].items():
        assert orc.retrieve_compression_config(cfgs, float(mb)) == layers
    with pytest.raises(ValueError) as e:
        orc.retrieve_compression_config(cfgs, 1)
    assert str(e.value) == g["too_small_error"]


def test_memory_per_block_constants():
    # bytes per block quoted for the 8B- and 70B-shaped projections
    assert orc.memory_per_block(4096, 4096) == 2359296
    assert orc.memory_per_block(1024, 4096) == 688128
    assert orc.memory_per_block(14336, 4096) == 7929856
    assert orc.memory_per_block(4096, 14336) == 7929856
    assert orc.memory_per_block(8192, 8192) == 8912896
    assert orc.memory_per_block(28672, 8192) == 30539776
