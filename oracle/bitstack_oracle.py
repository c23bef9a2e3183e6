"""CPU oracle for the BitStack residual-block linear layer.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
module; it is the checker that the CUDA path is compared against (tests, the
smoke entry and the CPU-baseline legs of the benchmark).

It restates, in plain numpy / torch-CPU code, the algorithm of the reference
operator:

* sign packing / unpacking       bitstack/utils/pack_utils.py:5-26
* per-block weight composition   bitstack/modules/BitStackLinear.py:7-15
* the unfused forward (level 0)  bitstack/modules/BitStackLinear.py:105-114
* offline decomposition          bitstack/modules/BitStackLinear.py:49-75
* bytes of one residual block    bitstack/modules/BitStackLinear.py:159-171
* budget lookup                  bitstack/utils/model_utils.py:179-187

Parity status: the reference stores no golden vectors for this path.  The
restatement is pinned against fixtures produced by running the reference's own
Python code on seeded inputs (tests/golden/make_golden.py wrote them; the
fixtures travel, the reference does not), plus the one known-answer vector the
packing convention implies (signs [+1,-1*7,-1*7,+1] -> bytes [128, 1]).
"""
from __future__ import annotations

import numpy as np

try:  # torch is only needed for the fp16-semantics restatement and decomposition
    import torch
except Exception:  # pragma: no cover - numpy-only use is still possible
    torch = None


# ----------------------------------------------------------------------------
# integer work: must be bit exact
# ----------------------------------------------------------------------------
def pack_sign(sign: np.ndarray) -> np.ndarray:
    """+1 -> bit 1, -1 -> bit 0; row-major flatten; 8 signs per byte, the first
    sign in the most significant bit; zero bits pad the last byte.
    Follows bitstack/utils/pack_utils.py:5-18."""
    s = np.asarray(sign)
    if not np.all(np.abs(s) == 1):
        raise AssertionError("pack_sign expects only +1 / -1")
    bits = ((s.astype(np.int16) + 1) // 2).astype(np.uint8).reshape(-1)
    pad = (-bits.size) % 8
    if pad:
        bits = np.concatenate([bits, np.zeros(pad, dtype=np.uint8)])
    bits = bits.reshape(-1, 8)
    weights = (1 << (7 - np.arange(8))).astype(np.uint8)
    return (bits * weights).sum(axis=1).astype(np.uint8)


def unpack_sign(packed: np.ndarray, shape) -> np.ndarray:
    """Inverse of pack_sign: int8 array of +1/-1 with the given shape; padding
    bits are dropped.  Follows bitstack/utils/pack_utils.py:20-26."""
    p = np.asarray(packed, dtype=np.uint8).reshape(-1, 1)
    masks = np.array([128, 64, 32, 16, 8, 4, 2, 1], dtype=np.uint8)
    bits = ((p & masks) > 0).astype(np.int8).reshape(-1)
    n = int(np.prod(shape))
    return (bits[:n] * 2 - 1).astype(np.int8).reshape(shape)


def memory_per_block(out_features: int, in_features: int, k: int = 16) -> int:
    """Bytes one residual block occupies: packed signs + fp16 u + fp16 vt.
    Follows bitstack/modules/BitStackLinear.py:159-171."""
    return (out_features * in_features) // 8 + 2 * k * (out_features + in_features)


def algorithmic_bytes(out_features, in_features, blocks, rows, k=16, bias=False) -> int:
    """Bytes a forward has to touch at least once: active blocks, x and y."""
    b = blocks * memory_per_block(out_features, in_features, k)
    b += 2 * rows * (in_features + out_features)
    if bias:
        b += 2 * out_features
    return b


# ----------------------------------------------------------------------------
# exact restatement (float64): the "what the stored data means" answer
# ----------------------------------------------------------------------------
def reconstruct_f64(qweight, u, vt, blocks, out_features, in_features) -> np.ndarray:
    """W = sum_j S_j * (U_j @ Vt_j) in float64 from stored tensors.
    qweight: (nb, M*N/8) u8, u: (nb, M, k) f16, vt: (nb, k, N) f16."""
    w = np.zeros((out_features, in_features), dtype=np.float64)
    for j in range(blocks):
        s = unpack_sign(qweight[j], (out_features, in_features)).astype(np.float64)
        w += s * (np.asarray(u[j], dtype=np.float64) @ np.asarray(vt[j], dtype=np.float64))
    return w


def forward_f64(x, qweight, u, vt, blocks, bias=None) -> np.ndarray:
    """y = x @ W^T (+ bias) in float64."""
    out_features, in_features = u.shape[1], vt.shape[2]
    w = reconstruct_f64(qweight, u, vt, blocks, out_features, in_features)
    y = np.asarray(x, dtype=np.float64) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y


def forward_f64_rows(x, qweight, u, vt, blocks, row_idx, bias=None) -> np.ndarray:
    """forward_f64 restricted to the output features in `row_idx` (cheap check at
    full benchmark sizes)."""
    row_idx = np.asarray(row_idx)
    m, n = u.shape[1], vt.shape[2]
    w = np.zeros((row_idx.size, n), dtype=np.float64)
    row_bytes_ok = (n % 8 == 0)
    for j in range(blocks):
        if row_bytes_ok:
            bits = np.unpackbits(np.asarray(qweight[j]).reshape(m, n // 8)[row_idx], axis=1)
            s = bits.astype(np.float64) * 2 - 1
        else:
            s = unpack_sign(qweight[j], (m, n))[row_idx].astype(np.float64)
        w += s * (np.asarray(u[j], dtype=np.float64)[row_idx] @ np.asarray(vt[j], dtype=np.float64))
    y = np.asarray(x, dtype=np.float64) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)[row_idx]
    return y


# ----------------------------------------------------------------------------
# fp16-semantics restatement of the reference's unfused forward (torch CPU)
# ----------------------------------------------------------------------------
def _t(a):
    if torch is None:
        raise RuntimeError("torch is required for the fp16 oracle")
    return a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))


def unpack_sign_t(packed, shape):
    """torch version of unpack_sign (same convention), used inside forward_l0."""
    packed = _t(packed)
    masks = torch.tensor([128, 64, 32, 16, 8, 4, 2, 1], dtype=torch.uint8)
    bits = ((packed.reshape(-1, 1) & masks) > 0).to(torch.int8).reshape(-1)
    n = 1
    for d in shape:
        n *= int(d)
    return bits[:n].reshape(tuple(shape)) * 2 - 1


def compose_block(packed, u, vt, shape):
    """One block's weight in the factors' dtype: sign * (u @ vt).
    Follows bitstack/modules/BitStackLinear.py:7-15 (no_avd=False)."""
    u, vt = _t(u), _t(vt)
    s = unpack_sign_t(packed, shape)
    return s.to(u.dtype) * torch.matmul(u, vt)


def reconstruct_l0(qweight, u, vt, blocks):
    """fp16 weight as level 0 builds it: zero fp16 matrix, one fp16 += per block.
    Follows bitstack/modules/BitStackLinear.py:107-113."""
    qweight, u, vt = _t(qweight), _t(u), _t(vt)
    m, n = u.shape[1], vt.shape[2]
    w = torch.zeros((m, n), dtype=torch.float16)
    for j in range(blocks):
        w += compose_block(qweight[j], u[j], vt[j], (m, n))
    return w


def forward_l0(x, qweight, u, vt, blocks, bias=None):
    """The reference's unfused forward on CPU: fp16 W, then F.linear in fp16.
    Follows bitstack/modules/BitStackLinear.py:105-114.  Returns a torch fp16
    tensor shaped like x with the last dim replaced by out_features."""
    x = _t(x)
    w = reconstruct_l0(qweight, u, vt, blocks)
    b = None if bias is None else _t(bias)
    with torch.no_grad():
        return torch.nn.functional.linear(x, w, b)


# ----------------------------------------------------------------------------
# offline decomposition (input generator for the "real weights" configuration)
# ----------------------------------------------------------------------------
def decompose_weight(weight, niter: int, k: int = 16):
    """Residual sign / rank-k decomposition.  Returns stacked
    (qweight u8 [niter, M*N/8], u f16 [niter, M, k], vt f16 [niter, k, N]).
    Follows bitstack/modules/BitStackLinear.py:49-75: zeros count as +1, the
    rank-k factors are U*sqrt(S) and sqrt(S)*Vt of |residual|, and the residual
    is updated with the un-rounded fp32 factors."""
    w = _t(weight).to(torch.float32).clone()
    m, n = w.shape
    qs, us, vts = [], [], []
    for _ in range(niter):
        sign = torch.sign(w)
        sign[sign == 0] = 1
        uu, ss, vv = torch.linalg.svd(w.abs(), full_matrices=False)
        root = torch.diag(torch.sqrt(ss[:k]))
        u_k = uu[:, :k] @ root
        vt_k = root @ vv[:k, :]
        packed = torch.from_numpy(pack_sign(sign.to(torch.int8).numpy()))
        qs.append(packed)
        us.append(u_k.to(torch.float16).contiguous())
        vts.append(vt_k.to(torch.float16).contiguous())
        w = w - sign * (u_k @ vt_k)
    return torch.stack(qs), torch.stack(us), torch.stack(vts)


# ----------------------------------------------------------------------------
# host logic restated for checking the loader
# ----------------------------------------------------------------------------
def retrieve_compression_config(configs, max_memory_mb):
    """Largest stored configuration whose 'memory' fits the budget.
    Follows bitstack/utils/model_utils.py:179-187."""
    limit = max_memory_mb * 1024 ** 2
    for cfg in sorted(configs, key=lambda c: c["memory"], reverse=True):
        if cfg["memory"] <= limit:
            return cfg["layers"]
    raise ValueError(f"No config found within the memory limit {max_memory_mb} MB")


def generate_configs(sorted_layer_bits, memory_per_bit, total_memory):
    """Cumulative one-block-at-a-time configurations.
    Follows bitstack/utils/model_utils.py:53-66."""
    layers = {name: 1 for name in memory_per_bit}
    out = [{"memory": total_memory, "layers": dict(layers)}]
    for name in sorted_layer_bits:
        total_memory += memory_per_bit[name]
        layers[name] += 1
        out.append({"memory": total_memory, "layers": dict(layers)})
    return out


# ----------------------------------------------------------------------------
# error metrics shared by every parity test
# ----------------------------------------------------------------------------
def max_normalised_error(got, ref) -> float:
    """max|got-ref| / max|ref| -- the form the 1e-2 output tolerance is applied in
    (element-wise relative error is meaningless on near-zero outputs)."""
    g = np.asarray(got, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    denom = np.max(np.abs(r))
    return float(np.max(np.abs(g - r)) / (denom if denom > 0 else 1.0))


def rel_l2_error(got, ref) -> float:
    g = np.asarray(got, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    denom = np.linalg.norm(r)
    return float(np.linalg.norm(g - r) / (denom if denom > 0 else 1.0))


# ----------------------------------------------------------------------------
# seeded synthetic inputs with the shapes / distributions of the benchmark configs
# ----------------------------------------------------------------------------
def synthetic_layer(out_features, in_features, blocks, seed, k=16, scale=0.05):
    """Bernoulli(0.5) packed signs, |N(0, scale)| fp16 factors (numpy arrays)."""
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 256, size=(blocks, (out_features * in_features) // 8), dtype=np.uint8)
    u = np.abs(rng.standard_normal((blocks, out_features, k)) * scale).astype(np.float16)
    vt = np.abs(rng.standard_normal((blocks, k, in_features)) * scale).astype(np.float16)
    return q, u, vt


def synthetic_input(rows, in_features, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((rows, in_features)).astype(np.float16)
