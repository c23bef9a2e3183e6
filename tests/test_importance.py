"""Block-importance scoring (bitstack/main.py:138-166 and the functions it uses, model_utils.py:26-51,117-133).

`tests/golden/importance.json` was produced by running the reference's own `sort_layers_and_bits_average` and
`eval_ppl` (tests/golden/make_importance_golden.py); the CPU tests pin this library's restatements to it, the
GPU test runs the whole loop on a small decoder and checks it against direct evaluations.
"""
import copy
import json
import math
import os

import pytest
import torch

from bitstack_b200 import importance, loader

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "importance.json")


def _golden():
    with open(GOLDEN) as f:
        return json.load(f)


def test_sort_order_matches_the_reference_function():
    for case in _golden()["sort_cases"]:
        given = copy.deepcopy(case["input"])
        assert importance.sort_layers_and_bits_average(given) == case["order"]
        # unlike the reference's, the restatement leaves its argument alone
        assert json.dumps(given) == json.dumps(case["input"])


def test_sort_rejects_a_missing_number_at_the_last_block_count():
    table = copy.deepcopy(_golden()["sort_cases"][0]["input"])
    table["reduced_ppl"][-1]["ppls"][0]["ppl"] = float("nan")
    with pytest.raises(ValueError, match="Last bit is nan"):
        importance.sort_layers_and_bits_average(table)


class _Table:
    def __init__(self, table):
        self.table = table

    def forward_logits(self, ids):
        return self.table[ids]


def test_perplexity_matches_the_reference_function():
    case = _golden()["ppl_case"]
    model = _Table(torch.tensor(case["table"]))
    ids = torch.tensor(case["ids"])
    got = importance.eval_ppl(case["batch_size"], model, ids)
    assert math.isclose(got, case["ppl"], rel_tol=1e-6), (got, case["ppl"])
    # the batch size only changes the grouping
    assert math.isclose(importance.eval_ppl(5, model, ids), case["ppl"], rel_tol=1e-6)


def test_order_feeds_the_budget_arithmetic():
    case = _golden()["sort_cases"][0]
    order = importance.sort_layers_and_bits_average(case["input"])
    names = sorted({e["layer"] for e in case["input"]["reduced_ppl"][0]["ppls"]})
    mem = {n: 1000 + 10 * i for i, n in enumerate(names)}
    cfgs = loader.generate_configs(order, mem, sum(mem.values()) + 500)
    assert len(cfgs) == len(order) + 1
    assert all(b["memory"] > a["memory"] for a, b in zip(cfgs, cfgs[1:]))
    assert cfgs[-1]["layers"] == {n: 4 for n in names}      # 3 scored block counts on top of the first block


@pytest.mark.gpu
def test_scoring_loop_on_a_small_decoder():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from bitstack_b200 import decode
    dev = torch.device("cuda:0")
    shape = decode.LlamaShape("tiny", 2, 512, 4, 2, 1024, vocab=1024)
    counts = {f"layer.{i}.{p}": 3 for i in range(2) for p in decode.PROJ_NAMES}
    model = decode.BitStackLlamaDecoder(shape, counts, dev, seed=3, max_len=64, batch=2)
    linears = model.bitstack_linears()
    assert [m.name for m in linears][:2] == ["layer.0.self_attn.q_proj", "layer.0.self_attn.k_proj"]
    linears[5].set_bit(2)                                   # a block count that must be put back afterwards
    g = torch.Generator(device=dev).manual_seed(1)
    calib = torch.randint(0, shape.vocab, (4, 32), device=dev, generator=g)
    seen = []
    table = importance.score_importance(model, calib, niter=3, batch_size=2, progress=lambda b, n, p: seen.append((b, n)))
    assert [m.w_bit for m in linears] == [3, 3, 3, 3, 3, 2, 3] + [3] * 7
    assert [b["bit"] for b in table["reduced_ppl"]] == [1, 2]
    assert all([e["layer"] for e in b["ppls"]] == [m.name for m in linears] for b in table["reduced_ppl"])
    assert len(seen) == 2 * len(linears)
    assert all(math.isfinite(e["ppl"]) and e["ppl"] > 1 for b in table["reduced_ppl"] for e in b["ppls"])
    # one entry against a direct evaluation, and the run is deterministic
    for m in linears:
        m.set_bit(2)
    linears[9].set_bit(3)
    direct = importance.eval_ppl(2, model, calib)
    assert direct == table["reduced_ppl"][1]["ppls"][9]["ppl"]
    for m in linears:
        m.set_bit(3)
    linears[5].set_bit(2)
    assert importance.eval_ppl(2, model, calib) == table["original_ppl"]
    again = importance.score_importance(model, calib, niter=3, batch_size=2)
    assert again == table
    # more blocks than are loaded
    with pytest.raises(ValueError):
        importance.score_importance(model, calib, niter=5, batch_size=2)
    # the forward used for scoring agrees with the decoder's own prefill on the last position
    logits = model.forward_logits(calib[:2])
    last = model._forward(calib[:2], model.arange[:32])
    assert torch.allclose(logits[:, -1].float(), last.float(), rtol=2e-2, atol=2e-3)
    order = importance.sort_layers_and_bits_average(table)
    mem = {m.name: m.memory_per_bit() for m in linears}
    cfgs = loader.generate_configs(order, mem, sum(mem.values()))
    assert cfgs[-1]["layers"] == {m.name: 3 for m in linears}
