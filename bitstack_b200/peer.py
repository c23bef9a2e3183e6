"""One-shot all-reduce over NVLink peer memory for the tensor-parallel decode step (C ABI: `bsb_peer_*`).

One process per GPU.  `PeerReduce(group, device, max_rows, max_width)` allocates this rank's area, exchanges the CUDA
inter-process handles through the process group (host side, set-up only) and maps the peers' areas;
`allreduce_add_rmsnorm` then replaces `all_reduce` + conversion + add/RMSNorm after a column-sharded projection with
one kernel per rank.  If peer mapping is not possible on the machine the constructor raises and the caller keeps NCCL.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


class PeerReduce:
    def __init__(self, group, device, max_rows: int, max_width: int):
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.max_rows, self.max_width = int(max_rows), int(max_width)
        lib = _lib.load()
        nbytes = lib.bsb_peer_area_bytes(self.world, self.max_rows, self.max_width)
        if nbytes < 0:
            raise ValueError(f"peer area: world {self.world}, rows {max_rows}, width {max_width} not supported")
        own, handle = C.c_void_p(), (C.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            _lib.check(lib.bsb_peer_alloc(nbytes, C.byref(own), handle), "bsb_peer_alloc")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self._areas = (C.c_void_p * self.world)()
            failed = None
            for p in range(self.world):
                if p == self.rank:
                    self._areas[p] = own.value
                    continue
                ptr = C.c_void_p()
                buf = (C.c_uint8 * 64).from_buffer_copy(handles[p])
                rc = lib.bsb_peer_open(buf, C.byref(ptr))
                if rc != 0:
                    failed = lib.bsb_last_error().decode(errors="replace")
                    break
                self._areas[p] = ptr.value
            # every rank must agree on whether the peer path is usable
            flags = [None] * self.world
            dist.all_gather_object(flags, failed, group=group)
            if any(f is not None for f in flags):
                self.close()
                raise _lib.BitStackLibraryError(f"peer mapping failed: {[f for f in flags if f]}")
        self._own = own.value

    def allreduce_add_rmsnorm(self, partial: torch.Tensor, h: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                              absmax: torch.Tensor = None) -> torch.Tensor:
        """partial: this rank's fp32 partial sums [rows, width]; h: fp16 residual stream [rows, width], updated in place
        with the all-reduced sum; returns rmsnorm(h) * norm_weight (fp16); `absmax` (fp32 [rows]) receives max |result|."""
        assert partial.dtype == torch.float32 and partial.is_cuda and partial.dim() == 2 and partial.stride(1) == 1
        rows, width = partial.shape
        assert h.dtype == torch.float16 and h.is_contiguous() and tuple(h.shape) == (rows, width)
        x = torch.empty_like(h)
        with torch.cuda.device(self.device):
            rc = _lib.load().bsb_peer_allreduce_add_rmsnorm(
                self._areas, self.rank, self.world, self.max_rows, self.max_width, partial.data_ptr(), partial.stride(0), rows,
                width, h.data_ptr(), norm_weight.data_ptr(), float(eps), x.data_ptr(),
                None if absmax is None else absmax.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "bsb_peer_allreduce_add_rmsnorm")
        return x

    def close(self):
        lib = _lib.load()
        areas = getattr(self, "_areas", None)
        if areas is None:
            return
        with torch.cuda.device(self.device):
            for p in range(self.world):
                if areas[p]:
                    lib.bsb_peer_close(areas[p], 1 if p == self.rank else 0)
                    areas[p] = None
        self._areas = None
