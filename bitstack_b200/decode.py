"""Greedy decode harness around the BitStack linear kernels.

The reference has no generation loop (its only model calls are full-sequence
forwards inside perplexity evaluation, bitstack/utils/model_utils.py:116-133), so
this is measurement scaffolding, not a mirror of reference code: a Llama-architecture
decoder (RMSNorm, rotary embedding, grouped-query attention over a static KV
cache, SwiGLU MLP) whose seven projections per layer are `BitStackLinear` modules
named like the reference names them (`layer.{i}.self_attn.q_proj`, ...,
bitstack/utils/decompose.py:14).  The glue ops are plain torch calls; one decode
step can be captured in a CUDA graph (device-side position and token feedback).

With `world_size > 1` the projections are sharded for tensor parallelism
(`bitstack_b200.sharding`): every rank draws the SAME full weight of a projection from the
seed and keeps its output rows (q/k/v/gate/up) or input columns (o/down), so the sharded
model computes what the single-device model computes.  The two column-sharded projections
of a layer deliver fp32 partial sums that are all-reduced and rounded to fp16 once; the LM
head is sharded by vocabulary (local maximum per rank, one small all-gather).
"""
from __future__ import annotations

import dataclasses
import random
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from . import glue
from . import _lib, sharding
from .linear import BitStackLinear, forward_grouped

PROJ_NAMES = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
              "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")


@dataclasses.dataclass
class LlamaShape:
    name: str
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    intermediate: int
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5

    @property
    def head_dim(self):
        return self.hidden // self.n_heads

    def proj_shapes(self) -> Dict[str, tuple]:
        kv = self.n_kv_heads * self.head_dim
        return {"self_attn.q_proj": (self.hidden, self.hidden), "self_attn.k_proj": (kv, self.hidden),
                "self_attn.v_proj": (kv, self.hidden), "self_attn.o_proj": (self.hidden, self.hidden),
                "mlp.gate_proj": (self.intermediate, self.hidden), "mlp.up_proj": (self.intermediate, self.hidden),
                "mlp.down_proj": (self.hidden, self.intermediate)}


LLAMA3_8B = LlamaShape("llama3-8b", 32, 4096, 32, 8, 14336)
LLAMA3_70B = LlamaShape("llama3-70b", 80, 8192, 64, 8, 28672)


def block_bytes(out_features, in_features, k=16):
    return (out_features * in_features) // 8 + 2 * k * (out_features + in_features)


def seeded_block_counts(shape: LlamaShape, seed: int, lo: int, hi: int, target_bytes: Optional[int] = None):
    """A compression config `{layer.i.proj: blocks}`: uniform draws in [lo, hi] from a
    seeded generator; when `target_bytes` is given, seeded single-block removals
    (never below `lo`) bring the packed total down to the target."""
    rng = random.Random(seed)
    shapes = shape.proj_shapes()
    names = [f"layer.{i}.{p}" for i in range(shape.n_layers) for p in PROJ_NAMES]
    counts = {n: rng.randint(lo, hi) for n in names}
    per_block = {n: block_bytes(*shapes[n.split(".", 2)[2]]) for n in names}
    if target_bytes is not None:
        total = sum(counts[n] * per_block[n] for n in names)
        while total > target_bytes:
            n = names[rng.randrange(len(names))]
            if counts[n] > lo:
                counts[n] -= 1
                total -= per_block[n]
            elif all(counts[m] <= lo for m in names):
                break
    return counts


def packed_bytes(shape: LlamaShape, counts: Dict[str, int]) -> int:
    shapes = shape.proj_shapes()
    return sum(c * block_bytes(*shapes[n.split(".", 2)[2]]) for n, c in counts.items())


COLUMN_SHARDED = ("self_attn.o_proj", "mlp.down_proj")   # input columns split over ranks: partial-sum outputs


def _random_bitstack(out_f, in_f, blocks, device, gen, name, fused_level, shard=None, rank=0, world=1):
    """Random-init module with the storage format of a loaded, stacked checkpoint:
    Bernoulli(0.5) packed signs, |N(0, 0.05)| fp16 factors.  `shard` ("rows" / "cols") with world > 1: the full
    weight is drawn (identically on every rank) and this rank's shard of it is kept."""
    q = torch.randint(0, 256, (blocks, out_f * in_f // 8), dtype=torch.uint8, device=device, generator=gen)
    u = (torch.randn(blocks, out_f, 16, device=device, generator=gen) * 0.05).abs().half()
    vt = (torch.randn(blocks, 16, in_f, device=device, generator=gen) * 0.05).abs().half()
    if world > 1 and shard == "rows":
        q, u, vt = sharding.shard_rows(q, u, vt, out_f, in_f, rank, world)
        out_f //= world
    elif world > 1 and shard == "cols":
        q, u, vt = sharding.shard_cols(q, u, vt, out_f, in_f, rank, world)
        in_f //= world
    m = BitStackLinear(w_bit=0, in_features=in_f, out_features=out_f, k=16, bias=False, no_avd=False,
                       dev=device, fused_level=fused_level)
    m.name = name
    m.qweight, m.u, m.vt = q, u, vt
    m.w_bit = blocks
    m._stacked_blocks = blocks
    return m


class BitStackLlamaDecoder:
    """Random-init Llama-architecture decoder whose linears are BitStack modules."""

    def __init__(self, shape: LlamaShape, block_counts: Dict[str, int], device, seed=0, max_len=1024,
                 batch=1, fused_level=6, rank=0, world_size=1, group=None, fused_glue=True, peer_reduce=True):
        self.shape, self.device, self.max_len, self.batch = shape, torch.device(device), max_len, batch
        self.fused_glue = fused_glue
        self.rank, self.world, self.group = rank, world_size, group
        # tensor parallel decode: the all-reduce after o / down as one kernel over NVLink peer memory (peer.py), fused
        # with the add + RMSNorm that follows; NCCL when the peers' memory cannot be mapped or the batch is too large
        self.peer = None
        if world_size > 1 and peer_reduce and batch <= 16:
            try:
                from .peer import PeerReduce
                self.peer = PeerReduce(group, self.device, max_rows=batch, max_width=shape.hidden)
            except Exception as e:   # noqa: BLE001 - any set-up failure means "use NCCL"
                self.peer_error = str(e)
        s = shape
        assert s.n_kv_heads % world_size == 0 and s.intermediate % (128 * world_size) == 0 and s.vocab % world_size == 0
        gen = torch.Generator(device=self.device).manual_seed(seed)  # same seed on every rank: replicated tensors agree
        self.embed = (torch.randn(s.vocab, s.hidden, device=self.device, generator=gen) * 0.02).half()
        lm_head = (torch.randn(s.vocab, s.hidden, device=self.device, generator=gen) * 0.02).half()
        # the head is sharded by vocabulary: rank p scores tokens [p V/P, (p+1) V/P)
        self.vocab_local = s.vocab // world_size
        self.lm_head = lm_head[rank * self.vocab_local:(rank + 1) * self.vocab_local].contiguous() if world_size > 1 else lm_head
        del lm_head
        self.final_norm = torch.ones(s.hidden, dtype=torch.float16, device=self.device)
        self.layers = []
        shapes = s.proj_shapes()
        W = world_size
        for i in range(s.n_layers):
            lay = {"in_norm": torch.ones(s.hidden, dtype=torch.float16, device=self.device),
                   "post_norm": torch.ones(s.hidden, dtype=torch.float16, device=self.device)}
            for p in PROJ_NAMES:
                out_f, in_f = shapes[p]
                # one seed per projection, the same on every rank: all ranks cut their shard out of the same weight
                lgen = torch.Generator(device=self.device).manual_seed(seed * 1000003 + i * 16 + PROJ_NAMES.index(p))
                lay[p] = _random_bitstack(out_f, in_f, block_counts[f"layer.{i}.{p}"], self.device, lgen,
                                          f"layer.{i}.{p}", fused_level,
                                          shard="cols" if p in COLUMN_SHARDED else "rows", rank=rank, world=W)
            self.layers.append(lay)
        hd = s.head_dim
        self.kv_local = s.n_kv_heads // W
        self.q_local = s.n_heads // W
        self.k_cache = [torch.zeros(batch, self.kv_local, max_len, hd, dtype=torch.float16, device=self.device) for _ in range(s.n_layers)]
        self.v_cache = [torch.zeros(batch, self.kv_local, max_len, hd, dtype=torch.float16, device=self.device) for _ in range(s.n_layers)]
        inv_freq = 1.0 / (s.rope_theta ** (torch.arange(0, hd, 2, device=self.device, dtype=torch.float32) / hd))
        t = torch.arange(max_len, device=self.device, dtype=torch.float32)
        freqs = torch.outer(t, inv_freq)
        self.cos = torch.cat([freqs, freqs], dim=-1).cos().half()
        self.sin = torch.cat([freqs, freqs], dim=-1).sin().half()
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)      # next position to write
        self.tokens = torch.zeros(batch, dtype=torch.long, device=self.device)  # token fed to the next step
        self.arange = torch.arange(max_len, device=self.device)
        self._graph = None

    # ------------------------------------------------------------------ pieces
    def weight_bytes(self):
        return sum(l[p].qweight.numel() + 2 * l[p].u.numel() + 2 * l[p].vt.numel() for l in self.layers for p in PROJ_NAMES)

    @staticmethod
    def _rope(x, cos, sin):
        half = x.shape[-1] // 2
        rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
        return x * cos + rot * sin

    def _row_parallel(self, mod, x, x_absmax=None):
        """A column-sharded projection (o / down): on one device the plain forward; tensor parallel, fp32 partial sums
        of this rank's input columns, summed over the ranks and rounded to fp16 once."""
        if self.world == 1:
            return forward_grouped([mod], x, x_absmax=x_absmax)[0] if x_absmax is not None else mod(x)
        part = mod.forward_partial(x)
        torch.distributed.all_reduce(part, group=self.group)
        return part.half()

    def _next_token(self, logits):
        """Greedy token from this rank's vocabulary shard of the logits [B, V/P]: local maximum, one all-gather of
        (value, index) pairs, first index of the global maximum (as argmax over the whole vocabulary gives)."""
        val, idx = logits.float().max(dim=-1)
        idx = idx + self.rank * self.vocab_local
        pair = torch.stack([val, idx.float()], dim=-1)                     # [B, 2]; token ids < 2^24 are exact in fp32
        allp = torch.empty(self.world, *pair.shape, dtype=pair.dtype, device=pair.device)
        torch.distributed.all_gather_into_tensor(allp, pair, group=self.group)
        best = allp[..., 0].max(dim=0)                                      # max returns the first (lowest-rank) maximum
        return allp[..., 1].gather(0, best.indices.unsqueeze(0)).squeeze(0).long()

    def _layer(self, i, h, positions, pos_index, mask):
        """h: [B, T, hidden]; positions: [T] long tensor of absolute positions."""
        s, lay = self.shape, self.layers[i]
        B, T, _ = h.shape
        x = F.rms_norm(h, (s.hidden,), lay["in_norm"], s.rms_eps)
        q, k, v = forward_grouped([lay["self_attn.q_proj"], lay["self_attn.k_proj"], lay["self_attn.v_proj"]], x)
        hd = s.head_dim
        q = q.view(B, T, self.q_local, hd).transpose(1, 2)
        k = k.view(B, T, self.kv_local, hd).transpose(1, 2)
        v = v.view(B, T, self.kv_local, hd).transpose(1, 2)
        cos, sin = self.cos.index_select(0, positions), self.sin.index_select(0, positions)
        q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
        self.k_cache[i].index_copy_(2, pos_index, k)
        self.v_cache[i].index_copy_(2, pos_index, v)
        att = F.scaled_dot_product_attention(q, self.k_cache[i], self.v_cache[i], attn_mask=mask, enable_gqa=True)
        att = att.transpose(1, 2).reshape(B, T, self.q_local * hd)
        h = h + self._row_parallel(lay["self_attn.o_proj"], att)
        x = F.rms_norm(h, (s.hidden,), lay["post_norm"], s.rms_eps)
        g, u = forward_grouped([lay["mlp.gate_proj"], lay["mlp.up_proj"]], x)
        h = h + self._row_parallel(lay["mlp.down_proj"], F.silu(g) * u)
        return h

    def _forward(self, token_ids, positions):
        """token_ids: [B, T]; returns last-position logits [B, vocab] and advances nothing."""
        h = self.embed.index_select(0, token_ids.reshape(-1)).view(*token_ids.shape, -1)
        mask = (self.arange.view(1, -1) <= positions.view(-1, 1)).view(1, 1, positions.numel(), self.max_len)
        for i in range(self.shape.n_layers):
            h = self._layer(i, h, positions, positions, mask)
        h = F.rms_norm(h[:, -1], (self.shape.hidden,), self.final_norm, self.shape.rms_eps)
        return h @ self.lm_head.t()

    @torch.no_grad()
    def forward_logits(self, token_ids):
        """Logits of every position, [B, T, vocab], for token_ids [B, T] on the device (B <= the decoder's batch,
        T <= max_len; one device).  Uses the first B rows of the KV cache as scratch: call it before `prefill`, not
        between decode steps.  This is the forward the perplexity evaluations of the importance scoring run."""
        assert self.world == 1, "forward_logits runs on one device"
        B, T = token_ids.shape
        assert B <= self.batch and T <= self.max_len
        positions = self.arange[:T]
        h = self.embed.index_select(0, token_ids.reshape(-1)).view(B, T, -1)
        mask = (self.arange.view(1, -1) <= positions.view(-1, 1)).view(1, 1, T, self.max_len)
        full_k, full_v = self.k_cache, self.v_cache
        try:
            if B < self.batch:
                self.k_cache = [c[:B] for c in full_k]
                self.v_cache = [c[:B] for c in full_v]
            for i in range(self.shape.n_layers):
                h = self._layer(i, h, positions, positions, mask)
        finally:
            self.k_cache, self.v_cache = full_k, full_v
        h = F.rms_norm(h, (self.shape.hidden,), self.final_norm, self.shape.rms_eps)
        return h @ self.lm_head.t()

    def bitstack_linears(self):
        """The BitStack projections in checkpoint order (their `.name` is `layer.{i}.{projection}`)."""
        return [lay[p] for lay in self.layers for p in PROJ_NAMES]

    def _decode_fused(self):
        """One decode step (one new token per sequence) with the fused glue kernels: per layer
        12 launches instead of ~30.  Same math as `_forward` on a single position."""
        s = self.shape
        B = self.batch
        hd = s.head_dim
        h = self.embed.index_select(0, self.tokens).contiguous()            # [B, hidden], residual stream
        fused_att = hd in (64, 128) and self.max_len <= 8192
        mask = None if fused_att else (self.arange <= self.pos).view(1, 1, 1, self.max_len)
        if self.peer is not None:
            return self._decode_fused_peer(h, fused_att, mask)
        delta = None                                                         # output of the previous MLP, not yet added to h
        # the stand-alone row kernels deliver max |x| with x: the operand preparation of the next call need not scan x
        am = torch.empty(B, dtype=torch.float32, device=self.device) if B <= 6 else None
        for i, lay in enumerate(self.layers):
            qkv = [lay["self_attn.q_proj"], lay["self_attn.k_proj"], lay["self_attn.v_proj"]]
            q, k, v = forward_grouped(qkv, glue.add_rmsnorm(h, delta, lay["in_norm"], s.rms_eps, absmax=am), x_absmax=am)
            att = self._attention(i, q, k, v, fused_att, mask)
            o = self._row_parallel(lay["self_attn.o_proj"], att)
            g, u = forward_grouped([lay["mlp.gate_proj"], lay["mlp.up_proj"]],
                                   glue.add_rmsnorm(h, o, lay["post_norm"], s.rms_eps, absmax=am), x_absmax=am)
            a = glue.silu_mul(g, u, absmax=am)
            delta = self._row_parallel(lay["mlp.down_proj"], a, x_absmax=am)
        x = glue.add_rmsnorm(h, delta, self.final_norm, s.rms_eps)
        return x @ self.lm_head.t()

    def _attention(self, i, q, k, v, fused_att, mask):
        s, B, hd = self.shape, self.batch, self.shape.head_dim
        if fused_att:
            return glue.decode_attention(q, k, v, self.cos, self.sin, self.pos, self.k_cache[i], self.v_cache[i],
                                         self.q_local, self.kv_local, hd)
        glue.rope_cache(q, k, v, self.cos, self.sin, self.pos, self.k_cache[i], self.v_cache[i], self.q_local, self.kv_local, hd)
        return F.scaled_dot_product_attention(q.view(B, self.q_local, 1, hd), self.k_cache[i], self.v_cache[i],
                                              attn_mask=mask, enable_gqa=True).reshape(B, self.q_local * hd)

    def _decode_fused_peer(self, h, fused_att, mask):
        """Tensor-parallel decode step with the one-shot peer all-reduce: o and down deliver fp32 partial sums, one
        kernel per rank exchanges them over NVLink, adds them in rank order, updates the residual stream and
        normalises it for the next projection.  Same values as the NCCL path (sum in fp32, one rounding)."""
        s, B = self.shape, self.batch
        am = torch.empty(B, dtype=torch.float32, device=self.device) if B <= 6 else None
        x = glue.add_rmsnorm(h, None, self.layers[0]["in_norm"], s.rms_eps, absmax=am)
        for i, lay in enumerate(self.layers):
            q, k, v = forward_grouped([lay["self_attn.q_proj"], lay["self_attn.k_proj"], lay["self_attn.v_proj"]], x, x_absmax=am)
            att = self._attention(i, q, k, v, fused_att, mask)
            x = self.peer.allreduce_add_rmsnorm(lay["self_attn.o_proj"].forward_partial(att), h, lay["post_norm"], s.rms_eps, am)
            g, u = forward_grouped([lay["mlp.gate_proj"], lay["mlp.up_proj"]], x, x_absmax=am)
            nxt = self.layers[i + 1]["in_norm"] if i + 1 < len(self.layers) else self.final_norm
            x = self.peer.allreduce_add_rmsnorm(lay["mlp.down_proj"].forward_partial(glue.silu_mul(g, u)), h, nxt, s.rms_eps, am)
        return x @ self.lm_head.t()

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor):
        """prompt_ids: [B, T] on the device.  Fills the KV cache and sets the first decode token."""
        B, T = prompt_ids.shape
        positions = torch.arange(T, device=self.device)
        logits = self._forward(prompt_ids, positions)
        self.tokens.copy_(logits.argmax(-1) if self.world == 1 else self._next_token(logits))
        self.pos.fill_(T)
        return self.tokens.clone()

    @torch.no_grad()
    def decode_step(self):
        """One greedy token for every sequence; position and token feedback stay on the device."""
        if self.fused_glue:
            logits = self._decode_fused()
            if self.world == 1 and logits.dtype == torch.float16 and logits.dim() == 2 and logits.stride(1) == 1:
                return glue.greedy_step(logits, self.tokens, self.pos)
        else:
            logits = self._forward(self.tokens.view(-1, 1), self.pos)
        self.tokens.copy_(logits.argmax(-1) if self.world == 1 else self._next_token(logits))
        self.pos.add_(1)
        return self.tokens

    def capture(self, stream=None):
        """Capture decode_step in a CUDA graph (call after prefill and a few eager steps)."""
        stream = stream or torch.cuda.Stream(self.device)
        pos0, tok0 = self.pos.clone(), self.tokens.clone()
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):
                self.decode_step()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            self.decode_step()
        self.pos.copy_(pos0)
        self.tokens.copy_(tok0)
        self._graph = g
        return g

    @torch.no_grad()
    def step(self):
        if self._graph is not None:
            self._graph.replay()
        else:
            self.decode_step()
        return self.tokens

    @torch.no_grad()
    def generate(self, prompt_ids_host: torch.Tensor, steps: int, pinned_out: Optional[torch.Tensor] = None):
        """Host-facing greedy generation: prompt on the host, every generated token read
        back to the host before the next step is issued (the call a user makes).
        Returns a [B, steps] CPU tensor."""
        prompt = prompt_ids_host.to(self.device, non_blocking=True)
        self.prefill(prompt)
        out = pinned_out if pinned_out is not None else torch.empty(steps, self.batch, dtype=torch.long).pin_memory()
        for t in range(steps):
            toks = self.step()
            out[t].copy_(toks, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
        with torch.cuda.device(self.device):
            _lib.check_device_status()   # a kernel that gave up a wait would have produced NaN outputs: fail loudly
        return out[:steps].t().contiguous()
