"""BitStackLinear: the reference's module interface on top of the sm_100a kernels.

Mirrors bitstack/modules/BitStackLinear.py:27-195 of the reference: same
constructor, buffer names / shapes / dtypes (these are the checkpoint keys),
`from_linear`, `forward`, `set_bit` / `pop_one_bit` / `add_one_bit`,
`stack_blocks`, `memory_per_bit`.  Every `fused_level` the reference accepts
(0-5) runs the same fused CUDA path here -- the levels only differed in how the
reference staged its Triton kernels -- and extra levels pin one kernel:

    0-5, 6  automatic choice (decode kernel, two rows per pass, for <= 6 rows; fused sign-GEMM up to 16 rows;
            rebuild + tcgen05 GEMM above)
    7       shape-agnostic CUDA-core kernel
    9       rebuild fp16 weight + tcgen05 GEMM
    10      decode kernel (tcgen05, sign operand in tensor memory), any row count
    11      fused sign-GEMM, tcgen05 variant (signs applied to tcgen05 rank-16 products in shared memory; up to 64 rows)
    12      fused sign-GEMM, register variant (warp-level MMAs, nothing between the two MMAs leaves the registers)

Differences from the reference's levels that a caller can observe: level 5 there takes 3-D inputs only and ignores
the bias (bitstack/modules/BitStackLinear.py:150-157); here every level takes any leading shape and adds the bias.
Level 4's fp16 atomics make the reference non-deterministic; here the same call is bit-identical run to run.

There is no CPU path: inputs must be CUDA fp16 tensors.  `no_avd=True` (the
reference's ablation without sign matrices) is not supported.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn

from . import _lib
from .pack import pack_sign, unpack_sign

_LEVEL_TO_ALGO = {0: _lib.ALGO_AUTO, 1: _lib.ALGO_AUTO, 2: _lib.ALGO_AUTO, 3: _lib.ALGO_AUTO,
                  4: _lib.ALGO_AUTO, 5: _lib.ALGO_AUTO, 6: _lib.ALGO_AUTO,
                  7: _lib.ALGO_GENERAL, 9: _lib.ALGO_REBUILD_GEMM, 10: _lib.ALGO_GEMV_TC5, 11: _lib.ALGO_SIGN_GEMM,
                  12: _lib.ALGO_SIGN_GEMM_MMA}

# scratch memory per (device index, stream handle); grown on demand, never shrunk
_workspaces: dict = {}
# scratch tensors whose address a captured CUDA graph may hold: kept alive for the life of the process
_pinned_workspaces: list = []


def get_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A cached uint8 scratch tensor of at least `nbytes` for the current stream of `device`.

    A scratch tensor handed out while its stream is being captured has its address baked into the graph.  It is
    therefore never freed: when a later request on that stream needs more, a new tensor serves the new calls and the
    old one stays allocated for the graph's replays.  Growing during a capture is refused (the allocation would land
    in the graph's private pool): run the step once eagerly before capturing it."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ent = _workspaces.get(key)          # [tensor, seen_by_a_capture]
    capturing = torch.cuda.is_current_stream_capturing()
    if ent is None or ent[0].numel() < nbytes:
        if capturing:
            raise RuntimeError(f"the scratch buffer of this stream must grow to {nbytes} bytes during a graph capture; "
                               "run the same calls once outside the capture first")
        if ent is not None and ent[1]:
            _pinned_workspaces.append(ent[0])
        ent = [torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device), False]
        _workspaces[key] = ent
    if capturing:
        ent[1] = True
    return ent[0]


@torch.no_grad()
def truncated_svd(a, k, oversample=16, power_iters=4, generator=None):
    """Leading k singular triplets of the fp32 matrix `a` [m, n]: randomised range finder (k + oversample Gaussian
    probes) with `power_iters` re-orthogonalised subspace iterations, then an exact SVD of the small projected
    matrix.  Returns (U [m, k], S [k], Vt [k, n]).  |W| of a weight matrix has one dominant (Perron) direction and a
    slowly decaying rest, which is why a few power iterations are needed for the trailing ranks."""
    m, n = a.shape
    l = min(k + oversample, m, n)
    omega = torch.randn(n, l, device=a.device, dtype=a.dtype, generator=generator)
    q, _ = torch.linalg.qr(a @ omega)
    for _ in range(power_iters):
        z, _ = torch.linalg.qr(a.t() @ q)
        q, _ = torch.linalg.qr(a @ z)
    b = q.t() @ a                                     # [l, n]
    ub, s, vt = torch.linalg.svd(b, full_matrices=False)
    return (q @ ub)[:, :k].contiguous(), s[:k].contiguous(), vt[:k, :].contiguous()


class BitStackLinear(nn.Module):
    def __init__(self, w_bit, in_features, out_features, k, bias, no_avd, dev, fused_level=0):
        super().__init__()
        if no_avd:
            raise NotImplementedError("no_avd=True (ablation without sign matrices) is not supported")
        self.in_features = in_features
        self.out_features = out_features
        self.w_bit = w_bit
        self.k = k
        self.no_avd = no_avd
        self.fused_level = fused_level
        self.name = None
        self._stacked_blocks = 0   # number of blocks held in the stacked tensors
        self._vt_absmax = None
        self._vt_key = None
        self._desc = None
        for i in range(self.w_bit):
            self.register_buffer(f"qweight_{i}", torch.zeros((out_features * in_features) // 8, dtype=torch.uint8, device=dev))
            self.register_buffer(f"u_{i}", torch.zeros(out_features, self.k, dtype=torch.float16, device=dev))
            self.register_buffer(f"vt_{i}", torch.zeros(self.k, in_features, dtype=torch.float16, device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16, device=dev))
        else:
            self.bias = None

    # ------------------------------------------------------------------ offline
    @torch.no_grad()
    def decompose_weight(self, original_weight, svd="full", oversample=16, power_iters=4, seed=0):
        """Residual sign / rank-k decomposition on the device (same recipe as
        bitstack/modules/BitStackLinear.py:49-75): zeros count as +1, factors are
        U*sqrt(S), sqrt(S)*Vt of |residual|, the residual uses the fp32 factors.

        `svd="full"` is the reference's `torch.linalg.svd` of the whole matrix per block.  `svd="randomized"` takes
        only the leading k triplets with a randomised range finder and `power_iters` subspace iterations
        (`truncated_svd` below): the cost per block drops from a full decomposition to a few products with
        (k + oversample)-column matrices.  It is not bit-compatible with the full SVD (the factors differ in the
        last bits and possibly in sign per rank); tests/test_decompose.py measures what that does to the singular
        values, to the residual after every block and to the forward."""
        if svd not in ("full", "randomized"):
            raise ValueError("svd must be 'full' or 'randomized'")
        weight = original_weight.to(torch.float32)
        shape = weight.shape
        gen = None
        if svd == "randomized":
            gen = torch.Generator(device=weight.device)
            gen.manual_seed(seed)
        for i in range(self.w_bit):
            sign = weight.sign()
            sign[sign == 0] = 1
            if svd == "full":
                u, s, vt = torch.linalg.svd(weight.abs(), full_matrices=False)
                u, s, vt = u[:, : self.k], s[: self.k], vt[: self.k, :]
            else:
                u, s, vt = truncated_svd(weight.abs(), self.k, oversample=oversample, power_iters=power_iters, generator=gen)
            root = torch.diag(torch.sqrt(s))
            us_k = u @ root
            vt_k = root @ vt
            packed = pack_sign(sign.to(torch.int8))
            assert unpack_sign(packed, shape).equal(sign.to(torch.int8))
            setattr(self, f"qweight_{i}", packed)
            setattr(self, f"u_{i}", us_k.to(torch.float16).contiguous())
            setattr(self, f"vt_{i}", vt_k.to(torch.float16).contiguous())
            w_i = sign * (us_k @ vt_k)
            assert torch.isinf(w_i).sum() == 0
            assert torch.isnan(w_i).sum() == 0
            weight = weight - w_i

    @classmethod
    def from_linear(cls, linear, w_bit, k=1, bias=True, no_avd=False, fused_level=0, name=None, init_only=False,
                    svd="full", **svd_options):
        qlinear = cls(w_bit=w_bit, in_features=linear.in_features, out_features=linear.out_features, bias=bias,
                      k=k, no_avd=no_avd, dev=linear.weight.device, fused_level=fused_level)
        qlinear.name = name
        if init_only:
            return qlinear
        qlinear.decompose_weight(linear.weight, svd=svd, **svd_options)
        if bias:
            qlinear.bias = linear.bias.detach().to(torch.float16)
        return qlinear

    def _load_from_state_dict(self, *args, **kwargs):
        # new buffer contents: everything derived from them is recomputed on the next forward
        super()._load_from_state_dict(*args, **kwargs)
        self._vt_absmax = None
        self._desc = None

    # ---------------------------------------------------------------- block count
    @property
    def blocks_loaded(self):
        """Blocks held in memory (set_bit may choose any count up to this one)."""
        return self._stacked_blocks if self._stacked_blocks else self.w_bit

    def pop_one_bit(self):
        self.w_bit -= 1

    def add_one_bit(self):
        self.w_bit += 1

    def set_bit(self, bit):
        self.w_bit = bit

    def memory_per_bit(self):
        """Bytes of one residual block: packed signs + u + vt."""
        return (self.out_features * self.in_features) // 8 + 2 * self.k * (self.out_features + self.in_features)

    # ------------------------------------------------------------------- stacking
    def _has_block_buffers(self):
        return "u_0" in self._buffers or hasattr(self, "u_0")

    def stack_blocks(self):
        """Per-block buffers -> stacked tensors `qweight [nb, out*in/8]`, `u [nb, out, k]`,
        `vt [nb, k, in]` (plain attributes); the per-block buffers are removed."""
        nb = self.w_bit
        self.qweight = torch.stack([getattr(self, f"qweight_{i}") for i in range(nb)])
        self.u = torch.stack([getattr(self, f"u_{i}") for i in range(nb)])
        self.vt = torch.stack([getattr(self, f"vt_{i}") for i in range(nb)])
        i = 0
        while hasattr(self, f"u_{i}"):
            delattr(self, f"qweight_{i}")
            delattr(self, f"u_{i}")
            delattr(self, f"vt_{i}")
            i += 1
        self._stacked_blocks = nb
        self._vt_absmax = None
        self._desc = None

    def _stack_keeping_buffers(self):
        """Level-0 style modules keep their per-block buffers (checkpoint keys); the
        kernels need one base pointer and a block stride, so the buffers are
        re-pointed at slices of one stacked allocation (no second copy is kept)."""
        nb = 0
        while hasattr(self, f"u_{nb}"):
            nb += 1
        q = torch.stack([getattr(self, f"qweight_{i}") for i in range(nb)])
        u = torch.stack([getattr(self, f"u_{i}") for i in range(nb)])
        vt = torch.stack([getattr(self, f"vt_{i}") for i in range(nb)])
        for i in range(nb):
            setattr(self, f"qweight_{i}", q[i])
            setattr(self, f"u_{i}", u[i])
            setattr(self, f"vt_{i}", vt[i])
        self.qweight, self.u, self.vt = q, u, vt
        self._stacked_blocks = nb
        self._vt_absmax = None
        self._desc = None

    def _buffers_alias_stack(self):
        if self._stacked_blocks == 0 or not hasattr(self, "u_0"):
            return self._stacked_blocks > 0
        n = self._stacked_blocks
        if hasattr(self, f"u_{n}"):
            return False
        for i in range(n):
            if (getattr(self, f"qweight_{i}").data_ptr() != self.qweight[i].data_ptr()
                    or getattr(self, f"u_{i}").data_ptr() != self.u[i].data_ptr()
                    or getattr(self, f"vt_{i}").data_ptr() != self.vt[i].data_ptr()):
                return False
        return True

    def _ensure_ready(self, device):
        if hasattr(self, "u_0"):
            if not self._buffers_alias_stack():
                self._stack_keeping_buffers()
        elif self._stacked_blocks == 0:
            if not hasattr(self, "qweight"):
                raise RuntimeError("BitStackLinear has neither per-block buffers nor stacked tensors")
            self._stacked_blocks = self.u.shape[0]
        if self.qweight.device != device:
            raise ValueError(f"input on {device} but weights on {self.qweight.device}")
        # max |vt| sets the scale of the decode kernel's fp8 operand: it must follow the CONTENT of vt, so the cache is
        # keyed on the tensor's version counter (bumped by every in-place write: copy_, load_state_dict, ...)
        try:
            version = self.vt._version
        except RuntimeError:        # inference-mode tensors keep no version counter: recompute on every call
            version = object()
        vt_key = (self.vt.data_ptr(), version, self._stacked_blocks)
        if self._vt_absmax is None or self._vt_absmax.device != device or self._vt_key != vt_key:
            self._vt_key = vt_key
            self._desc = None
            self._vt_absmax = torch.empty(self._stacked_blocks, self.k, dtype=torch.float32, device=device)
            if self.k == 16 and self._stacked_blocks > 0:
                d = self._make_desc(self._stacked_blocks, with_absmax=False)
                with torch.cuda.device(device):
                    _lib.check(_lib.load().bsb_vt_absmax(C.byref(d), self._vt_absmax.data_ptr(),
                                                         torch.cuda.current_stream(device).cuda_stream), "vt_absmax")

    def _make_desc(self, blocks, with_absmax=True):
        d = _lib.BsbWeight()
        d.qweight = self.qweight.data_ptr()
        d.u = self.u.data_ptr()
        d.vt = self.vt.data_ptr()
        d.bias = self.bias.data_ptr() if self.bias is not None else None
        d.vt_absmax = self._vt_absmax.data_ptr() if (with_absmax and self.k == 16 and self._vt_absmax is not None) else None
        d.q_block_stride = self.qweight.stride(0) if self.qweight.dim() > 1 else self.qweight.numel()
        d.u_block_stride = self.u.stride(0)
        d.vt_block_stride = self.vt.stride(0)
        d.out_features, d.in_features, d.k, d.blocks = self.out_features, self.in_features, self.k, blocks
        return d

    def weight_desc(self, device=None):
        """The `bsb_weight` descriptor for the current active block count."""
        device = device or self.qweight.device
        self._ensure_ready(device)
        if self.w_bit < 0 or self.w_bit > self._stacked_blocks:
            raise ValueError(f"w_bit={self.w_bit} but only {self._stacked_blocks} blocks are loaded")
        key = (self.w_bit, self.qweight.data_ptr(), self.u.data_ptr(), self.vt.data_ptr(),
               None if self.bias is None else self.bias.data_ptr(), self._vt_absmax.data_ptr())
        if self._desc is None or self._desc[0] != key:
            self._desc = (key, self._make_desc(self.w_bit))
        return self._desc[1]

    # -------------------------------------------------------------------- forward
    @torch.no_grad()
    def reconstruct_weight(self):
        """fp16 [out, in] weight of the active blocks (products rounded to fp16 and summed in fp16 like the reference's
        reconstruction, last block first; the general kernel for ragged shapes sums in fp32)."""
        dev = self.qweight.device if hasattr(self, "qweight") else self.u_0.device
        d = self.weight_desc(dev)
        w = torch.empty(self.out_features, self.in_features, dtype=torch.float16, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().bsb_reconstruct_weight(C.byref(d), w.data_ptr(),
                                                          torch.cuda.current_stream(dev).cuda_stream), "reconstruct_weight")
        return w

    @torch.no_grad()
    def forward_partial(self, x):
        """Tensor-parallel variant of `forward`: the product as fp32 partial sums (no rounding to fp16), for a module
        that holds an input-column shard of a projection; the caller all-reduces and rounds once."""
        return self.forward(x, _partial=True)

    @torch.no_grad()
    def forward(self, x, _partial=False):
        if self.fused_level not in _LEVEL_TO_ALGO:
            raise ValueError(f"Invalid fused_level: {self.fused_level}")
        if not x.is_cuda:
            raise ValueError("BitStackLinear (B200) needs CUDA inputs; there is no CPU path")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"last input dim {x.shape[-1]} != in_features {self.in_features}")
        algo = _LEVEL_TO_ALGO[self.fused_level]
        x16 = x if x.dtype == torch.float16 else x.to(torch.float16)
        x2 = x16.reshape(-1, self.in_features)
        if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < self.in_features):
            x2 = x2.contiguous()
        rows = x2.shape[0]
        d = self.weight_desc(x.device)
        y = torch.empty(rows, self.out_features, dtype=torch.float32 if _partial else torch.float16, device=x.device)
        lib = _lib.load()
        with torch.cuda.device(x.device):
            need = lib.bsb_linear_workspace_bytes(C.byref(d), rows, algo)
            if need < 0:
                raise ValueError("bsb_linear_workspace_bytes rejected the arguments: " + lib.bsb_last_error().decode())
            ws = get_workspace(x.device, need)
            fn = lib.bsb_linear_forward_partial if _partial else lib.bsb_linear_forward
            rc = fn(C.byref(d), x2.data_ptr(), rows, x2.stride(0) if rows > 1 else self.in_features,
                    y.data_ptr(), self.out_features, ws.data_ptr(), ws.numel(), algo,
                    torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc, "bsb_linear_forward")
        return y.reshape(*x.shape[:-1], self.out_features)


def forward_grouped(modules, x, algo=_lib.ALGO_AUTO, *, x_absmax=None):
    """Apply several BitStackLinear modules to the same input with one fused launch
    sequence (q/k/v or gate/up of a decoder layer).  Returns a list of outputs.

    `x_absmax` (fp32 [rows], decode path only: rows <= 6): max |x| per row as the producer of x delivered it
    (`glue.add_rmsnorm` / `glue.silu_mul`), so that the operand preparation does not scan x for it."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    n = len(modules)
    descs = (_lib.BsbWeight * n)()
    for i, m in enumerate(modules):
        src = m.weight_desc(x.device)
        C.memmove(C.byref(descs[i]), C.byref(src), C.sizeof(_lib.BsbWeight))
    ys = [torch.empty(rows, m.out_features, dtype=torch.float16, device=x.device) for m in modules]
    yptrs = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    ystr = (C.c_int64 * n)(*[m.out_features for m in modules])
    lib = _lib.load()
    with torch.cuda.device(x.device):
        need = lib.bsb_linear_grouped_workspace_bytes(descs, n, rows, algo)
        if need < 0:
            raise ValueError("grouped workspace query rejected the arguments: " + lib.bsb_last_error().decode())
        ws = get_workspace(x.device, need)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        xs = x2.stride(0) if rows > 1 else x2.shape[-1]
        if x_absmax is None:
            rc = lib.bsb_linear_forward_grouped(descs, n, x2.data_ptr(), rows, xs, yptrs, ystr, ws.data_ptr(), ws.numel(),
                                                algo, stream)
        else:
            assert x_absmax.dtype == torch.float32 and x_absmax.is_cuda and x_absmax.numel() >= rows
            rc = lib.bsb_linear_forward_grouped_ex(descs, n, x2.data_ptr(), rows, xs, x_absmax.data_ptr(), yptrs, ystr,
                                                   ws.data_ptr(), ws.numel(), stream)
    _lib.check(rc, "bsb_linear_forward_grouped")
    return [y.reshape(*x.shape[:-1], m.out_features) for y, m in zip(ys, modules)]
