"""Block-importance scoring on the fused path: which projection gains most from one more residual block.

Mirrors the scoring loop of the reference's driver (bitstack/main.py:138-166) and the two functions around it
(`eval_ppl`, bitstack/utils/model_utils.py:117-133; `sort_layers_and_bits_average`, model_utils.py:26-51), so
that the table it writes (`reduced_ppl_average.json`) and the order derived from it feed the budget arithmetic
(`loader.generate_configs`) exactly as the reference's do.

What makes the loop cheap here: the number of active blocks is a kernel argument (`set_bit` moves no data), and
every perplexity evaluation is a batch forward on the tensor-core batch path.  The model is anything with

    forward_logits(ids [B, T] on the device) -> logits [B, T, vocab]
    bitstack_linears() -> list of BitStackLinear modules whose `.name` is the checkpoint's layer name

(`decode.BitStackLlamaDecoder` has both).  The calibration text is the caller's: token ids [n_sequences, T].
"""
from __future__ import annotations

import json
import math
from typing import Callable, Dict, List, Optional

import torch


@torch.no_grad()
def eval_ppl(batch_size: int, model, input_ids: torch.Tensor) -> float:
    """Perplexity as the reference measures it (model_utils.py:117-133): next-token cross entropy averaged per
    sequence, then over sequences, exponentiated."""
    nlls = []
    for i in range(0, len(input_ids), batch_size):
        ids = input_ids[i:i + batch_size]
        logits = model.forward_logits(ids)
        shift_logits = logits[:, :-1, :].float()
        shift_labels = ids[:, 1:]
        loss = torch.nn.functional.cross_entropy(shift_logits.permute(0, 2, 1), shift_labels, reduction="none")
        nlls.append(loss.float().mean(dim=1))
    return float(torch.exp(torch.cat(nlls).mean()).item())


@torch.no_grad()
def score_importance(model, calib_ids: torch.Tensor, niter: int, batch_size: int = 4,
                     save_path: Optional[str] = None, progress: Optional[Callable[[int, str, float], None]] = None) -> Dict:
    """For every block count `bit` in 1 .. niter-1: all projections at `bit` blocks, then each projection alone at
    `bit + 1` — the perplexity it reaches is its score for that block (main.py:146-158).  Returns, and writes to
    `save_path` after every finished block count like the reference, the table
    {"original_ppl": p, "reduced_ppl": [{"bit": b, "ppls": [{"layer": name, "ppl": p}, ...]}, ...]}.
    The projections' block counts are put back to what they were."""
    linears = model.bitstack_linears()
    before = [m.w_bit for m in linears]
    for m in linears:
        if m.blocks_loaded < niter:
            raise ValueError(f"{m.name}: {m.blocks_loaded} blocks loaded, scoring up to {niter} needs {niter}")
    try:
        original = eval_ppl(batch_size, model, calib_ids)
        table = {"original_ppl": original, "reduced_ppl": []}
        for bit in range(1, niter):
            for m in linears:
                m.set_bit(bit)
            ppls = []
            for m in linears:
                m.set_bit(bit + 1)
                p = eval_ppl(batch_size, model, calib_ids)
                if progress is not None:
                    progress(bit, m.name, p)
                ppls.append({"layer": m.name, "ppl": p})
                m.set_bit(bit)
            table["reduced_ppl"].append({"bit": bit, "ppls": ppls})
            if save_path is not None:
                with open(save_path, "w") as f:
                    json.dump(table, f, indent=4)
    finally:
        for m, b in zip(linears, before):
            m.set_bit(b)
    return table


def _is_nan(v) -> bool:
    return isinstance(v, float) and math.isnan(v) or str(v).lower() == "nan"


def sort_layers_and_bits_average(data: Dict) -> List[str]:
    """Order in which blocks are added to the budget (model_utils.py:26-51): per block count, projections by
    ascending perplexity; an entry without a number takes the next block count's perplexity of the same projection
    plus this block count's largest one, so that it sorts behind the measured ones.  `data` is not modified."""
    bits = [{"bit": b["bit"], "ppls": [dict(p) for p in b["ppls"]]} for b in data["reduced_ppl"]]
    max_bit = len(bits)
    for bit in reversed(range(max_bit)):
        ppls = bits[bit]["ppls"]
        # Python's max over floats with NaNs depends on their position; the reference takes it as is
        max_ppl = max(ppls, key=lambda x: x["ppl"])["ppl"]
        if _is_nan(max_ppl):
            max_ppl = 0
        for idx, entry in enumerate(ppls):
            if _is_nan(entry["ppl"]):
                if bit == max_bit - 1:
                    raise ValueError("Last bit is nan")
                nxt = bits[bit + 1]["ppls"]
                assert nxt[idx]["layer"] == entry["layer"]
                entry["ppl"] = nxt[idx]["ppl"] + max_ppl
    order: List[str] = []
    for b in range(max_bit):
        order.extend(e["layer"] for e in sorted(bits[b]["ppls"], key=lambda x: x["ppl"]))
    return order
