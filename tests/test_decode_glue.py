"""GPU checks of the fused decode glue kernels against plain torch fp32 references, and of the
fused decode step against the unfused torch-op step of the same harness."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _seed():
    """Every test draws its random inputs from the same seed: greedy tokens of a random-init model sit on near-ties,
    so an unseeded prompt makes the token comparisons below depend on the draw."""
    torch.manual_seed(20241)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(20241)


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (3, 8192), (16, 128)])
def test_add_rmsnorm(dev, rows, hidden):
    from bitstack_b200 import glue
    g = torch.Generator(device=dev).manual_seed(rows + hidden)
    h = torch.randn(rows, hidden, device=dev, generator=g).half()
    d = torch.randn(rows, hidden, device=dev, generator=g).half()
    w = (1 + 0.1 * torch.randn(hidden, device=dev, generator=g)).half()
    h_ref = (h.float() + d.float()).half()
    y_ref = (h_ref.float() * torch.rsqrt(h_ref.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())
    h2 = h.clone()
    y = glue.add_rmsnorm(h2, d, w, 1e-5)
    assert torch.equal(h2, h_ref)
    assert (y.float() - y_ref).abs().max() <= 2e-3 * y_ref.abs().max()
    h3 = h.clone()
    y0 = glue.add_rmsnorm(h3, None, w, 1e-5)
    assert torch.equal(h3, h)
    ref0 = h.float() * torch.rsqrt(h.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert (y0.float() - ref0).abs().max() <= 2e-3 * ref0.abs().max()


def test_silu_mul(dev):
    from bitstack_b200 import glue
    g = torch.randn(4, 14336, device=dev).half()
    u = torch.randn(4, 14336, device=dev).half()
    out = glue.silu_mul(g, u)
    ref = F.silu(g.float()) * u.float()
    assert (out.float() - ref).abs().max() <= 4e-3 * ref.abs().max()


def test_rope_cache(dev):
    from bitstack_b200 import glue
    B, Hq, Hkv, D, L = 2, 8, 2, 128, 64
    q = torch.randn(B, Hq * D, device=dev).half()
    k = torch.randn(B, Hkv * D, device=dev).half()
    v = torch.randn(B, Hkv * D, device=dev).half()
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(L, device=dev).float(), inv)
    cos, sin = torch.cat([fr, fr], -1).cos().half(), torch.cat([fr, fr], -1).sin().half()
    kc = torch.zeros(B, Hkv, L, D, device=dev, dtype=torch.float16)
    vc = torch.zeros_like(kc)
    pos = torch.tensor([37], device=dev)

    def rope(x, heads):
        x = x.view(B, heads, D).float()
        rot = torch.cat([-x[..., D // 2:], x[..., :D // 2]], -1)
        return x * cos[37].float() + rot * sin[37].float()

    q_ref, k_ref = rope(q, Hq), rope(k, Hkv)
    glue.rope_cache(q, k, v, cos, sin, pos, kc, vc, Hq, Hkv, D)
    assert (q.view(B, Hq, D).float() - q_ref).abs().max() <= 4e-3 * q_ref.abs().max()
    assert (kc[:, :, 37].float() - k_ref).abs().max() <= 4e-3 * k_ref.abs().max()
    assert torch.equal(vc[:, :, 37], v.view(B, Hkv, D))
    assert kc[:, :, :37].abs().max() == 0 and kc[:, :, 38:].abs().max() == 0


@pytest.mark.parametrize("B,Hq,Hkv,D,L,at", [(2, 8, 2, 128, 64, 37), (1, 32, 8, 128, 700, 640), (3, 4, 4, 64, 40, 0), (1, 8, 1, 128, 33, 32)])
def test_decode_attention_matches_rope_then_sdpa(dev, B, Hq, Hkv, D, L, at):
    """Fused rotary + cache write + single-token attention against the separate rotary kernel followed by
    torch's scaled_dot_product_attention on the same caches."""
    from bitstack_b200 import glue
    g = torch.Generator(device=dev).manual_seed(B * 1000 + at)
    q = torch.randn(B, Hq * D, device=dev, generator=g).half()
    k = torch.randn(B, Hkv * D, device=dev, generator=g).half()
    v = torch.randn(B, Hkv * D, device=dev, generator=g).half()
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device=dev).float() / D))
    fr = torch.outer(torch.arange(L, device=dev).float(), inv)
    cos, sin = torch.cat([fr, fr], -1).cos().half(), torch.cat([fr, fr], -1).sin().half()
    kc = torch.randn(B, Hkv, L, D, device=dev, generator=g).half()
    vc = torch.randn(B, Hkv, L, D, device=dev, generator=g).half()
    kc[:, :, at:] = 0
    vc[:, :, at:] = 0
    pos = torch.tensor([at], device=dev)
    kc2, vc2, q2 = kc.clone(), vc.clone(), q.clone()
    out = glue.decode_attention(q, k, v, cos, sin, pos, kc, vc, Hq, Hkv, D)
    assert torch.equal(q, q2)                                  # q is not modified
    glue.rope_cache(q2, k, v, cos, sin, pos, kc2, vc2, Hq, Hkv, D)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)        # same cache contents, bit for bit
    mask = (torch.arange(L, device=dev) <= at).view(1, 1, 1, L)
    ref = F.scaled_dot_product_attention(q2.view(B, Hq, 1, D).float(), kc2.float(), vc2.float(), attn_mask=mask,
                                         enable_gqa=True).reshape(B, Hq * D)
    assert (out.float() - ref).abs().max() <= 3e-3 * ref.abs().max()


def test_decode_harness_small_batch_under_a_cuda_graph(dev):
    """Batch 3 (row pairs + a single row in every projection), captured as a CUDA graph and replayed: same tokens and
    logits as the eager unfused path."""
    from bitstack_b200 import decode
    shape = decode.LlamaShape("tiny", 2, 512, 4, 2, 1024, vocab=1000)
    counts = decode.seeded_block_counts(shape, seed=4, lo=2, hi=4)
    prompt = torch.randint(0, 1000, (3, 7), device=dev, generator=torch.Generator(device=dev).manual_seed(2))
    ref = decode.BitStackLlamaDecoder(shape, counts, dev, seed=6, max_len=128, batch=3, fused_glue=False)
    ref.prefill(prompt)
    want = [ref.decode_step().clone() for _ in range(5)]
    m = decode.BitStackLlamaDecoder(shape, counts, dev, seed=6, max_len=128, batch=3, fused_glue=True)
    m.prefill(prompt)
    m.capture()
    got = [m.step().clone() for _ in range(5)]
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(want, got)), (want, got)


def test_greedy_step_is_argmax_with_first_index_ties(dev):
    from bitstack_b200 import glue
    g = torch.Generator(device=dev).manual_seed(9)
    for B, V in ((1, 128256), (3, 1000), (2, 7), (4, 32000)):
        logits = torch.randn(B, V, device=dev, generator=g).half()
        logits[0, V // 2] = 9.0
        logits[0, V - 1] = 9.0          # tie: the lower index wins
        if B > 1:
            logits[1, 0] = 11.0
        tokens = torch.zeros(B, dtype=torch.long, device=dev)
        pos = torch.tensor([41], device=dev)
        glue.greedy_step(logits, tokens, pos)
        assert torch.equal(tokens, logits.float().argmax(-1)) and tokens[0].item() == V // 2
        assert pos.item() == 42
        # a view with a row stride larger than the vocabulary, no position update
        wide = torch.zeros(B, V + 8, device=dev, dtype=torch.float16)
        wide[:, :V] = logits
        glue.greedy_step(wide[:, :V], tokens.zero_(), None)
        assert torch.equal(tokens, logits.float().argmax(-1))


def test_fused_decode_step_matches_unfused(dev):
    from bitstack_b200 import decode
    shape = decode.LlamaShape("tiny", 2, 512, 4, 2, 1024, vocab=1000)
    counts = decode.seeded_block_counts(shape, seed=3, lo=2, hi=4)
    prompt = torch.randint(0, 1000, (1, 9), device=dev)
    outs = []
    for fused in (False, True):
        m = decode.BitStackLlamaDecoder(shape, counts, dev, seed=5, max_len=128, fused_glue=fused)
        m.prefill(prompt)
        toks, logits = [], None
        for _ in range(4):
            logits = (m._decode_fused() if fused else m._forward(m.tokens.view(-1, 1), m.pos)).float()
            m.tokens.copy_(logits.argmax(-1))
            m.pos.add_(1)
            toks.append(int(m.tokens[0]))
        outs.append((toks, logits))
    (t0, l0) = outs[0]
    for t1, l1 in outs[1:]:
        assert (l0 - l1).abs().max() <= 2e-2 * l0.abs().max()
        assert t0 == t1


@pytest.mark.parametrize("rows", [1, 2, 5])
def test_row_kernels_deliver_the_row_maximum_and_the_projection_call_takes_it(dev, rows):
    """The stand-alone row kernels (add + rmsnorm, silu * up) also deliver max |result| per row; a projection call that
    is handed that number gives bit-identical outputs to one that scans x itself."""
    from bitstack_b200 import forward_grouped, glue
    from bitstack_b200.layer_bench import synthetic_projection
    N, M = 1024, 768
    g = torch.Generator(device=dev).manual_seed(rows)
    h = torch.randn(rows, N, device=dev, generator=g).half()
    d = torch.randn(rows, N, device=dev, generator=g).half()
    w = (1 + 0.1 * torch.randn(N, device=dev, generator=g)).half()
    am = torch.zeros(rows, dtype=torch.float32, device=dev)
    h1, h2 = h.clone(), h.clone()
    x = glue.add_rmsnorm(h1, d, w, 1e-5, absmax=am)
    assert torch.equal(x, glue.add_rmsnorm(h2, d, w, 1e-5)) and torch.equal(h1, h2)
    assert torch.equal(am, x.float().abs().amax(dim=1))
    mods = [synthetic_projection(M, N, 3, 10, dev, seed=1), synthetic_projection(256, N, 2, 10, dev, seed=2)]
    for a, b in zip(forward_grouped(mods, x, x_absmax=am), forward_grouped(mods, x)):
        assert torch.equal(a, b)
    gate = torch.randn(rows, N, device=dev, generator=g).half()
    up = torch.randn(rows, N, device=dev, generator=g).half()
    am2 = torch.zeros(rows, dtype=torch.float32, device=dev)
    a = glue.silu_mul(gate, up, absmax=am2)
    assert torch.equal(a, glue.silu_mul(gate, up)) and torch.equal(am2, a.float().abs().amax(dim=1))
    want = (torch.nn.functional.silu(gate) * up).float()
    assert (a.float() - want).abs().max() <= 2e-3 * want.abs().max()
