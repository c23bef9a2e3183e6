"""Fused decode-time glue ops (residual add + RMSNorm, rotary + KV-cache write, SiLU*up) on CUDA
tensors, through the C ABI.  These are harness helpers around the BitStack projections; the
reference leaves the same ops to the Hugging Face Llama modules."""
from __future__ import annotations

import torch

from . import _lib


_att_scratch = {}   # (device, batch, heads, head_dim) -> zero-initialised scratch of decode_attention


def _s(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def add_rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float, absmax: torch.Tensor = None) -> torch.Tensor:
    """In place h += delta (skipped when delta is None); returns rmsnorm(h) * weight.  h: [rows, hidden] fp16.
    `absmax` (fp32 [rows], optional) receives max |result| per row."""
    assert h.is_cuda and h.dtype == torch.float16 and h.is_contiguous() and h.dim() == 2
    if delta is not None:
        delta = delta.reshape(h.shape)
        assert delta.dtype == torch.float16 and delta.is_contiguous()
    if absmax is not None:
        assert absmax.dtype == torch.float32 and absmax.is_contiguous() and absmax.numel() >= h.shape[0]
    y = torch.empty_like(h)
    with torch.cuda.device(h.device):
        rc = _lib.load().bsb_add_rmsnorm(h.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                         float(eps), y.data_ptr(), None if absmax is None else absmax.data_ptr(),
                                         h.shape[0], h.shape[1], _s(h))
    _lib.check(rc, "bsb_add_rmsnorm")
    return y


def rope_cache(q, k, v, cos, sin, pos, k_cache, v_cache, q_heads, kv_heads, head_dim):
    """Rotary embedding at position pos[0] (device int64) on q in place and on k, which goes with v
    into k_cache / v_cache [batch, kv_heads, max_len, head_dim]."""
    for t in (q, k, v, cos, sin, k_cache, v_cache):
        assert t.is_cuda and t.dtype == torch.float16 and t.is_contiguous()
    assert pos.dtype == torch.int64 and pos.is_cuda
    batch = q.shape[0]
    with torch.cuda.device(q.device):
        rc = _lib.load().bsb_rope_cache(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                        pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), batch, q_heads, kv_heads,
                                        head_dim, k_cache.shape[2], _s(q))
    _lib.check(rc, "bsb_rope_cache")
    return q


def decode_attention(q, k, v, cos, sin, pos, k_cache, v_cache, q_heads, kv_heads, head_dim):
    """One new token per batch row: rotary embedding of q and k at position pos[0] (device int64), k and v
    appended to k_cache / v_cache [batch, kv_heads, max_len, head_dim], then grouped-query attention of the
    rotated q over cache positions 0..pos.  q is left untouched; returns [batch, q_heads * head_dim] fp16."""
    for t in (q, k, v, cos, sin, k_cache, v_cache):
        assert t.is_cuda and t.dtype == torch.float16 and t.is_contiguous()
    assert pos.dtype == torch.int64 and pos.is_cuda
    batch = q.shape[0]
    out = torch.empty(batch, q_heads * head_dim, dtype=torch.float16, device=q.device)
    lib = _lib.load()
    key = (q.device.index, batch, q_heads, head_dim)
    scratch = _att_scratch.get(key)
    if scratch is None:   # zeroed once; the kernel leaves its counters at zero for the next call
        scratch = torch.zeros(lib.bsb_decode_attention_scratch_bytes(batch, q_heads, head_dim), dtype=torch.uint8, device=q.device)
        _att_scratch[key] = scratch
    with torch.cuda.device(q.device):
        rc = lib.bsb_decode_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                      pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), batch,
                                      q_heads, kv_heads, head_dim, k_cache.shape[2], scratch.data_ptr(), scratch.numel(), _s(q))
    _lib.check(rc, "bsb_decode_attention")
    return out


def greedy_step(logits: torch.Tensor, tokens: torch.Tensor, pos) -> torch.Tensor:
    """tokens[b] = argmax(logits[b]) (first maximum), then pos[0] += 1 (skipped when pos is None), in one launch.
    logits: [batch, vocab] fp16 with unit inner stride; tokens: [batch] int64; pos: [1] int64 or None."""
    assert logits.is_cuda and logits.dtype == torch.float16 and logits.dim() == 2 and logits.stride(1) == 1
    assert tokens.dtype == torch.int64 and tokens.is_contiguous() and tokens.numel() == logits.shape[0]
    assert pos is None or (pos.dtype == torch.int64 and pos.is_cuda)
    with torch.cuda.device(logits.device):
        rc = _lib.load().bsb_greedy_step(logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0), tokens.data_ptr(),
                                         None if pos is None else pos.data_ptr(), _s(logits))
    _lib.check(rc, "bsb_greedy_step")
    return tokens


def silu_mul(gate: torch.Tensor, up: torch.Tensor, absmax: torch.Tensor = None) -> torch.Tensor:
    """silu(gate) * up on [rows, n] fp16 (n % 8 == 0); `absmax` (fp32 [rows], optional) receives max |result| per row."""
    assert gate.is_cuda and gate.dtype == torch.float16 and gate.is_contiguous() and up.is_contiguous()
    g2 = gate.reshape(-1, gate.shape[-1])
    out = torch.empty_like(gate)
    with torch.cuda.device(gate.device):
        rc = _lib.load().bsb_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(),
                                      None if absmax is None else absmax.data_ptr(), g2.shape[0], g2.shape[1], _s(gate))
    _lib.check(rc, "bsb_silu_mul")
    return out
