"""Tensor-parallel sharding of stacked BitStack weights (pure tensor slicing; device agnostic).

The reference has no tensor parallelism (its only multi-GPU mode is layer placement by
accelerate, bitstack/utils/model_utils.py:198), so the contract here is "same math as one
device":

* output-row shard (q/k/v/gate/up): rank p keeps rows [p*M/P, (p+1)*M/P) of every sign
  matrix and of U; Vt is replicated.  Packed bytes of a row range are contiguous.
* input-column shard (o/down): rank p keeps columns [p*N/P, (p+1)*N/P): a strided byte
  gather of the packed signs (N/P must be a multiple of 8; the tensor-core kernels need a
  multiple of 128), the matching columns of Vt; U is replicated.  Outputs are partial sums
  and must be all-reduced.
"""
from __future__ import annotations

import torch


def shard_rows(qweight, u, vt, out_features, in_features, rank, world):
    """qweight [nb, M*N/8] u8, u [nb, M, k], vt [nb, k, N] -> this rank's row shard."""
    if out_features % world:
        raise ValueError(f"out_features {out_features} not divisible by world size {world}")
    rows = out_features // world
    if (rows * in_features) % 8:
        raise ValueError("a row shard must cover whole packed bytes")
    lo = rank * rows
    row_bytes = in_features // 8
    q = qweight.view(qweight.shape[0], out_features, row_bytes)[:, lo:lo + rows].reshape(qweight.shape[0], -1)
    return q.contiguous(), u[:, lo:lo + rows].contiguous(), vt.contiguous()


def shard_cols(qweight, u, vt, out_features, in_features, rank, world):
    """-> this rank's input-column shard (partial-sum outputs)."""
    if in_features % (8 * world):
        raise ValueError(f"in_features {in_features} must be a multiple of 8*world_size")
    cols = in_features // world
    lo = rank * cols
    row_bytes = in_features // 8
    q = qweight.view(qweight.shape[0], out_features, row_bytes)[:, :, lo // 8:(lo + cols) // 8]
    return q.reshape(qweight.shape[0], -1).contiguous(), u.contiguous(), vt[:, :, lo:lo + cols].contiguous()
