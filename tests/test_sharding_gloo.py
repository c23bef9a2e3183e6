"""Tensor-parallel sharding arithmetic on CPU ranks (gloo, world size 2): row shards
concatenate, column shards all-reduce, both must reproduce the single-device oracle."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import bitstack_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bitstack_b200.sharding import shard_cols, shard_rows
    m, n, nb = 64, 256, 3
    q, u, vt = orc.synthetic_layer(m, n, nb, seed=9)
    x = orc.synthetic_input(2, n, seed=10)
    full = orc.forward_f64(x, q, u, vt, nb)
    tq, tu, tvt = torch.from_numpy(q), torch.from_numpy(u), torch.from_numpy(vt)
    # output-row shard: each rank owns a slice of the outputs
    rq, ru, rvt = shard_rows(tq, tu, tvt, m, n, rank, world)
    y_rows = orc.forward_f64(x, rq.numpy(), ru.numpy(), rvt.numpy(), nb)
    gathered = [torch.zeros(2, m // world, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y_rows))
    err_rows = float(np.abs(torch.cat(gathered, dim=1).numpy() - full).max())
    # input-column shard: partial sums, one all-reduce
    cq, cu, cvt = shard_cols(tq, tu, tvt, m, n, rank, world)
    lo = rank * (n // world)
    part = torch.from_numpy(orc.forward_f64(x[:, lo:lo + n // world], cq.numpy(), cu.numpy(), cvt.numpy(), nb))
    dist.all_reduce(part)
    err_cols = float(np.abs(part.numpy() - full).max())
    # the packed bytes of a column shard are exactly the shard of the unpacked signs
    s_full = orc.unpack_sign(q[0], (m, n))[:, lo:lo + n // world]
    same_bits = bool(np.array_equal(orc.unpack_sign(cq[0].numpy(), (m, n // world)), s_full))
    if rank == 0:
        out_q.put((err_rows, err_cols, same_bits, float(np.abs(full).max())))
    dist.barrier()
    dist.destroy_process_group()


def test_row_and_column_shards_match_single_device():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    err_rows, err_cols, same_bits, scale = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same_bits
    assert err_rows <= 1e-12 * scale
    assert err_cols <= 1e-9 * scale


def test_shard_argument_errors():
    import pytest
    from bitstack_b200.sharding import shard_cols, shard_rows
    q = torch.zeros(1, 6 * 24 // 8, dtype=torch.uint8)
    u, vt = torch.zeros(1, 6, 16, dtype=torch.float16), torch.zeros(1, 16, 24, dtype=torch.float16)
    with pytest.raises(ValueError):
        shard_rows(q, u, vt, 6, 24, 0, 4)
    with pytest.raises(ValueError):
        shard_cols(q, u, vt, 6, 24, 0, 2)
