"""Tensor parallelism on hardware: the 2-rank decoder (NCCL, one process per GPU) against the single-device decoder.

Every rank cuts its shards (`sharding.shard_rows` / `shard_cols`) out of the SAME seeded full weights, so the sharded
model must compute what one device computes: the column-sharded projections deliver fp32 partial sums that are
all-reduced and rounded once, the head is sharded by vocabulary.  Asserted: identical greedy tokens over several steps
and last-step logits equal to fp16 rounding.  Skipped with fewer than two GPUs.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, peer, out_q):
    import datetime
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    from bitstack_b200 import decode
    shape = decode.LlamaShape("tiny", 2, 1024, 8, 4, 2048, vocab=2048)
    counts = decode.seeded_block_counts(shape, seed=4, lo=2, hi=5)
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, shape.vocab, (batch, 9), generator=gen).to(dev)
    tp = decode.BitStackLlamaDecoder(shape, counts, dev, seed=6, max_len=128, batch=batch, rank=rank, world_size=world,
                                     group=dist.group.WORLD, peer_reduce=peer)
    assert (tp.peer is not None) == peer, getattr(tp, "peer_error", None)
    tp.prefill(prompt)
    toks = []
    for _ in range(5):
        toks.append(tp.decode_step().clone())
    logits_local = tp._decode_fused().float()                      # [B, V / world]
    gathered = [torch.empty_like(logits_local) for _ in range(world)]
    dist.all_gather(gathered, logits_local)
    logits = torch.cat(gathered, dim=-1)
    if rank == 0:
        one = decode.BitStackLlamaDecoder(shape, counts, dev, seed=6, max_len=128, batch=batch)
        one.prefill(prompt)
        want = [one.decode_step().clone() for _ in range(5)]
        ref_logits = one._decode_fused().float()
        same = all(torch.equal(a, b) for a, b in zip(toks, want))
        err = float((logits - ref_logits).abs().max() / ref_logits.abs().max())
        out_q.put((same, err, [t.tolist() for t in toks], [t.tolist() for t in want]))
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)    # skip the communicator destructors (they were seen to block at exit after graph / PDL work)


@pytest.mark.parametrize("peer", [False, True])
@pytest.mark.parametrize("batch", [1, 3])
def test_two_rank_decoder_matches_one_device(batch, peer):
    """peer=False: NCCL all-reduce of the fp32 partials; peer=True: the one-shot all-reduce over NVLink peer memory fused
    with the add + RMSNorm (`bsb_peer_allreduce_add_rmsnorm`)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, peer, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, err, got, want = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert same, (got, want)
    assert err <= 4e-3, err
