"""Pins the decode harness to a real Llama: Hugging Face's `LlamaForCausalLM` (fp32) built from the SAME tensors --
embedding, head, norm weights, and every projection's weight reconstructed from the BitStack blocks -- must give the
logits and greedy tokens of `BitStackLlamaDecoder` (rotary convention and theta, grouped-query head grouping, norm
placement, SwiGLU order, residual order).  The reference wraps exactly these Hugging Face modules
(bitstack/utils/decompose.py:7-21 replaces the linears inside `model.model.layers`)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decoder_matches_huggingface_llama_built_from_the_same_tensors():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    transformers = pytest.importorskip("transformers")
    from bitstack_b200 import decode
    dev = torch.device("cuda:0")
    shape = decode.LlamaShape("tiny", 2, 512, 4, 2, 1024, vocab=1000)
    counts = decode.seeded_block_counts(shape, seed=4, lo=2, hi=4)
    m = decode.BitStackLlamaDecoder(shape, counts, dev, seed=6, max_len=128, batch=1)
    g = torch.Generator(device=dev).manual_seed(1)
    for lay in m.layers:       # non-trivial norm weights, so that their placement matters
        for k in ("in_norm", "post_norm"):
            lay[k] = (1 + 0.2 * torch.randn(shape.hidden, device=dev, generator=g)).half()
    m.final_norm = (1 + 0.2 * torch.randn(shape.hidden, device=dev, generator=g)).half()

    cfg = transformers.LlamaConfig(hidden_size=shape.hidden, intermediate_size=shape.intermediate, num_hidden_layers=shape.n_layers,
                                   num_attention_heads=shape.n_heads, num_key_value_heads=shape.n_kv_heads, vocab_size=shape.vocab,
                                   rms_norm_eps=shape.rms_eps, rope_theta=shape.rope_theta, max_position_embeddings=128,
                                   tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    hf = transformers.LlamaForCausalLM(cfg).to(dev).float().eval()
    sd = {"model.embed_tokens.weight": m.embed.float(), "lm_head.weight": m.lm_head.float(), "model.norm.weight": m.final_norm.float()}
    for i, lay in enumerate(m.layers):
        sd[f"model.layers.{i}.input_layernorm.weight"] = lay["in_norm"].float()
        sd[f"model.layers.{i}.post_attention_layernorm.weight"] = lay["post_norm"].float()
        for p in decode.PROJ_NAMES:
            sd[f"model.layers.{i}.{p}.weight"] = lay[p].reconstruct_weight().float()
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and all("rotary" in k or "inv_freq" in k for k in missing), (missing, unexpected)

    prompt = torch.randint(0, shape.vocab, (1, 11), device=dev, generator=g)
    with torch.no_grad():
        ref_logits = hf(prompt).logits[:, -1].float()
    ours = m._forward(prompt, torch.arange(prompt.shape[1], device=dev)).float()
    err = float((ours - ref_logits).abs().max() / ref_logits.abs().max())
    assert err <= 2e-2, err

    # greedy continuation: the harness (prefill, then fused decode steps on the KV cache) against full re-evaluation
    m.prefill(prompt)
    seq = prompt.clone()
    for _ in range(4):
        with torch.no_grad():
            lg = hf(seq).logits[0, -1].float()
        tok = int(m.tokens[0])                       # token the harness feeds next
        # the harness token must be Hugging Face's argmax, or tie with it within the fp16 noise of the logits
        assert lg[tok] >= lg.max() - 2e-2 * lg.abs().max(), (tok, int(lg.argmax()))
        seq = torch.cat([seq, torch.tensor([[tok]], device=dev)], dim=1)
        m.decode_step()
