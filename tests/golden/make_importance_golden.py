"""Generates tests/golden/importance.json by running the reference's own functions.

    python tests/golden/make_importance_golden.py /path/to/reference

`bitstack/utils/model_utils.py` cannot be imported here (it imports plotting / dispatch packages that are not
installed), so `sort_layers_and_bits_average` (model_utils.py:26-51) and `eval_ppl` (model_utils.py:117-133) are
compiled from its source text, unchanged, and run on small seeded inputs:

  sort cases   reduced-perplexity tables (one with NaN entries) -> the order in which blocks are added
  ppl case     seeded logits of a stand-in model on seeded token ids -> the perplexity eval_ppl reports
"""
import ast
import json
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _reference_functions(ref_root):
    path = os.path.join(ref_root, "bitstack", "utils", "model_utils.py")
    tree = ast.parse(open(path).read())
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("sort_layers_and_bits_average", "eval_ppl")]
    from tqdm import tqdm
    ns = {"torch": torch, "tqdm": tqdm}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), path, "exec"), ns)
    return ns["sort_layers_and_bits_average"], ns["eval_ppl"]


class _StandIn(torch.nn.Module):
    """Anything with `.eval()`, `.device` and a call returning an object with `.logits` serves eval_ppl."""

    def __init__(self, table):
        super().__init__()
        self.table = table          # [vocab, vocab]: logits of the next token given the current one
        self.device = torch.device("cpu")

    def forward(self, ids):
        return types.SimpleNamespace(logits=self.table[ids])


def main():
    ref_root = sys.argv[1]
    sort_fn, ppl_fn = _reference_functions(ref_root)
    g = torch.Generator().manual_seed(7)
    layers = [f"layer.{i}.{p}" for i in range(2) for p in ("self_attn.q_proj", "mlp.down_proj", "mlp.up_proj")]
    cases = []
    for case in range(2):
        table = {"original_ppl": 10.0, "reduced_ppl": []}
        for bit in range(1, 4):
            ppls = [{"layer": l, "ppl": round(float(8 + 4 * torch.rand((), generator=g)), 4)} for l in layers]
            table["reduced_ppl"].append({"bit": bit, "ppls": ppls})
        if case == 1:   # NaN entries in the first two bits (the last bit must not hold one)
            table["reduced_ppl"][0]["ppls"][1]["ppl"] = float("nan")
            table["reduced_ppl"][0]["ppls"][4]["ppl"] = float("nan")
            table["reduced_ppl"][1]["ppls"][4]["ppl"] = float("nan")
        given = json.loads(json.dumps(table))          # the function edits its argument in place
        order = sort_fn(table)
        cases.append({"input": given, "order": order})
    vocab, nseq, seqlen = 17, 5, 9
    logits = torch.randn(vocab, vocab, generator=g)
    ids = torch.randint(0, vocab, (nseq, seqlen), generator=g)
    ppl = ppl_fn(2, seqlen, _StandIn(logits), ids, disable_tqdm=True)
    out = {"sort_cases": cases, "ppl_case": {"table": logits.tolist(), "ids": ids.tolist(), "batch_size": 2, "ppl": ppl}}
    with open(os.path.join(HERE, "importance.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("written", os.path.join(HERE, "importance.json"))


if __name__ == "__main__":
    main()
