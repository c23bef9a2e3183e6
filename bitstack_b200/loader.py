"""Memory-budget loading of BitStack checkpoints, written against the safetensors file format directly.

Mirrors the reference's loading path (bitstack/utils/model_utils.py:179-205 and
bitstack/utils/decompose.py:7-21) without `accelerate`:

* `retrieve_compression_config(configs, max_memory_MB)` and `generate_configs(...)` have the reference's
  names, arguments, results and error (model_utils.py:53-66, 179-187).  `configs` is the list stored
  in a checkpoint's `compression_config.json`: `[{"memory": bytes, "layers": {"layer.3.self_attn.q_proj": 5, ...}}, ...]`.
* `load_bitstack_linears(..., rank, world)` places the packed blocks across devices for tensor parallelism: a rank
  reads only its output rows of q/k/v/gate/up (one contiguous byte range of every `qweight_j` and `u_j`) or its input
  columns of o/down (a strided cut of `qweight_j` and `vt_j`), as `bitstack_b200.sharding` defines them.  The reference
  places whole layers on devices through accelerate (model_utils.py:189-205); it has no tensor parallelism.
* `load_bitstack_linears(...)` builds one `BitStackLinear` per decomposed projection, named
  `layer.{i}.{sub}` as `decompose()` names them, and reads ONLY the first `nb` residual blocks of each
  (`qweight_{j}`, `u_{j}`, `vt_{j}`, j < nb: the checkpoint keys of bitstack/modules/BitStackLinear.py:38-46)
  straight into the stacked `[nb, ...]` tensors the kernels consume.  Raising the budget later means
  loading more blocks; lowering it is `set_bit()` and never repacks.

The file format: 8 bytes little-endian header length, a JSON header `{name: {"dtype", "shape",
"data_offsets": [begin, end]}, "__metadata__": ...}`, then the raw little-endian tensor bytes.  A
sharded checkpoint adds `model.safetensors.index.json` with `{"weight_map": {name: file}}`.
"""
from __future__ import annotations

import json
import os
import re
import struct
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import numpy as np
import torch

from . import sharding
from .linear import BitStackLinear

_DTYPES = {
    "U8": (np.uint8, torch.uint8), "I8": (np.int8, torch.int8), "F16": (np.float16, torch.float16),
    "F32": (np.float32, torch.float32), "I32": (np.int32, torch.int32), "I64": (np.int64, torch.int64),
    "BF16": (np.uint16, torch.bfloat16),
}
_NAMES = {torch.uint8: "U8", torch.int8: "I8", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32",
          torch.int64: "I64", torch.bfloat16: "BF16"}


# ----------------------------------------------------------------------------- budget arithmetic
def retrieve_compression_config(configs, max_memory_MB):
    """The largest stored configuration that fits `max_memory_MB` MiB: its `layers` dict
    (model_utils.py:179-187).  Raises ValueError when none fits, as the reference does."""
    max_memory = max_memory_MB * 1024 ** 2
    for config in sorted(configs, key=lambda c: c["memory"], reverse=True):
        if config["memory"] <= max_memory:
            return config["layers"]
    raise ValueError(f"No config found within the memory limit {max_memory_MB} MB")


def generate_configs(sorted_layer_bits, memory_per_bit, total_memory):
    """All budget steps from "every layer one block" upwards, adding blocks in the given order
    (model_utils.py:53-66).  `total_memory` starts as one block per layer plus the non-BitStack memory."""
    configs = []
    layers = {layer: 1 for layer in memory_per_bit.keys()}
    configs.append({"memory": total_memory, "layers": layers.copy()})
    for layer in sorted_layer_bits:
        total_memory += memory_per_bit[layer]
        layers[layer] += 1
        configs.append({"memory": total_memory, "layers": layers.copy()})
    return configs


def memory_per_block(out_features: int, in_features: int, k: int = 16) -> int:
    """Bytes of one residual block (bitstack/modules/BitStackLinear.py:159-171)."""
    return out_features * in_features // 8 + 2 * k * (out_features + in_features)


# ----------------------------------------------------------------------------- safetensors files
class SafetensorsFile:
    """Header of one .safetensors file plus ranged reads of its tensors."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
            (n,) = struct.unpack("<Q", head)
            if n <= 0 or n > (100 << 20):
                raise ValueError(f"{path}: implausible header length {n}")
            header = json.loads(f.read(n).decode("utf-8"))
        self.data_start = 8 + n
        self.metadata = header.pop("__metadata__", None)
        self.entries: Dict[str, dict] = header
        size = os.path.getsize(path)
        for name, e in self.entries.items():
            b, en = e["data_offsets"]
            if e["dtype"] not in _DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
            want = int(np.prod(e["shape"], dtype=np.int64)) * np.dtype(_DTYPES[e["dtype"]][0]).itemsize
            if not (0 <= b <= en and self.data_start + en <= size and en - b == want):
                raise ValueError(f"{path}: tensor {name} has inconsistent offsets {e['data_offsets']} for shape {e['shape']}")

    def keys(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self.entries[name]
        return _DTYPES[e["dtype"]][1], tuple(e["shape"])

    def read_into(self, name: str, dst: torch.Tensor) -> None:
        """Copies tensor `name` into `dst` (same dtype and element count; any device)."""
        e = self.entries[name]
        np_dt, t_dt = _DTYPES[e["dtype"]]
        if dst.dtype != t_dt or dst.numel() != int(np.prod(e["shape"], dtype=np.int64)):
            raise ValueError(f"{name}: checkpoint holds {e['dtype']}{e['shape']}, destination is {dst.dtype}{tuple(dst.shape)}")
        b, en = e["data_offsets"]
        if en == b:
            return
        raw = np.fromfile(self.path, dtype=np.uint8, count=en - b, offset=self.data_start + b)
        if raw.size != en - b:
            raise ValueError(f"{self.path}: short read of {name}")
        dst.copy_(torch.from_numpy(raw).view(t_dt).reshape(dst.shape), non_blocking=False)

    def read_rows_into(self, name: str, row_begin: int, row_end: int, dst: torch.Tensor) -> None:
        """Copies rows [row_begin, row_end) of tensor `name`, seen as a matrix whose first dimension has the stored
        tensor's leading extent (any trailing shape), into `dst`: one contiguous byte range of the file."""
        e = self.entries[name]
        np_dt, t_dt = _DTYPES[e["dtype"]]
        shape = e["shape"]
        n0 = int(shape[0]) if shape else 1
        total = int(np.prod(shape, dtype=np.int64))
        if not (0 <= row_begin <= row_end <= n0):
            raise ValueError(f"{name}: rows [{row_begin}, {row_end}) outside 0..{n0}")
        per_row = (total // n0) * np.dtype(np_dt).itemsize if n0 else 0
        nbytes = (row_end - row_begin) * per_row
        if dst.dtype != t_dt or dst.numel() * dst.element_size() != nbytes:
            raise ValueError(f"{name}: destination does not hold rows [{row_begin}, {row_end})")
        if nbytes == 0:
            return
        b = e["data_offsets"][0]
        raw = np.fromfile(self.path, dtype=np.uint8, count=nbytes, offset=self.data_start + b + row_begin * per_row)
        if raw.size != nbytes:
            raise ValueError(f"{self.path}: short read of {name}")
        dst.copy_(torch.from_numpy(raw).view(t_dt).reshape(dst.shape), non_blocking=False)

    def read(self, name: str, device="cpu") -> torch.Tensor:
        dt, shape = self.info(name)
        out = torch.empty(shape, dtype=dt, device=device)
        self.read_into(name, out)
        return out


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Writes `tensors` (CPU or CUDA, contiguous or not) as one .safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    blobs: List[bytes] = []
    off = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


class Checkpoint:
    """A directory of .safetensors shards (with or without an index file) seen as one name space."""

    def __init__(self, directory: str):
        self.directory = directory
        self._files: Dict[str, SafetensorsFile] = {}
        self.weight_map: Dict[str, str] = {}
        index = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                self.weight_map = dict(json.load(f)["weight_map"])
        else:
            shards = sorted(p for p in os.listdir(directory) if p.endswith(".safetensors"))
            if not shards:
                raise FileNotFoundError(f"no .safetensors file in {directory}")
            for shard in shards:
                for name in self._file(shard).keys():
                    self.weight_map[name] = shard

    def _file(self, shard: str) -> SafetensorsFile:
        if shard not in self._files:
            self._files[shard] = SafetensorsFile(os.path.join(self.directory, shard))
        return self._files[shard]

    def __contains__(self, name: str) -> bool:
        return name in self.weight_map

    def info(self, name: str):
        return self._file(self.weight_map[name]).info(name)

    def read_into(self, name: str, dst: torch.Tensor) -> None:
        if name not in self.weight_map:
            raise KeyError(f"{name} is not in the checkpoint at {self.directory}")
        self._file(self.weight_map[name]).read_into(name, dst)

    def read_rows_into(self, name: str, row_begin: int, row_end: int, dst: torch.Tensor) -> None:
        if name not in self.weight_map:
            raise KeyError(f"{name} is not in the checkpoint at {self.directory}")
        self._file(self.weight_map[name]).read_rows_into(name, row_begin, row_end, dst)

    def compression_configs(self):
        """The list stored by the reference in `compression_config.json` (main.py:168-184)."""
        with open(os.path.join(self.directory, "compression_config.json")) as f:
            return json.load(f)


# ----------------------------------------------------------------------------- the loader
_PROJ = re.compile(r"^(?P<prefix>.*layers)\.(?P<i>\d+)\.(?P<sub>.+)\.qweight_0$")


def discover_projections(ckpt: Checkpoint) -> Dict[str, str]:
    """{`layer.{i}.{sub}`: checkpoint key prefix} for every module that stores `qweight_0`."""
    found = {}
    for name in ckpt.weight_map:
        m = _PROJ.match(name)
        if m:
            found[f"layer.{m.group('i')}.{m.group('sub')}"] = f"{m.group('prefix')}.{m.group('i')}.{m.group('sub')}"
    return found


def stored_blocks(ckpt: Checkpoint, prefix: str) -> int:
    n = 0
    while f"{prefix}.qweight_{n}" in ckpt:
        n += 1
    return n


@torch.no_grad()
def load_bitstack_linears(directory: str, compression_config: Optional[Mapping[str, int]] = None, *, max_memory_MB=None,
                          niter: Optional[int] = None, k: int = 16, device="cuda", fused_level: int = 6,
                          names: Optional[Iterable[str]] = None, rank: int = 0, world: int = 1,
                          shard_rule=None) -> Dict[str, BitStackLinear]:
    """Builds the BitStack projections of a decomposed checkpoint with only the blocks the budget allows.

    Block counts come from `compression_config` ({`layer.{i}.{sub}`: blocks}), else from the checkpoint's
    `compression_config.json` and `max_memory_MB`, else `niter` blocks everywhere — the same precedence
    as `decompose(init_only=True)` (decompose.py:14-19).  Each module comes back stacked
    (`stack_blocks()` done: `qweight [nb, out*in/8]`, `u [nb, out, k]`, `vt [nb, k, in]`), named, and with
    `w_bit` = the loaded block count.

    `world > 1` places the blocks for tensor parallelism: this `rank` gets the output-row shard of a projection
    (`shard_rule(name) == "rows"`: a contiguous byte range of each `qweight_j` / `u_j` is read, nothing else of them
    touches memory) or its input-column shard (`"cols"`: partial-sum outputs, see `BitStackLinear.forward_partial`).
    The default rule shards `o_proj` / `down_proj` by columns and every other projection by rows; a rule may return
    None to keep a projection whole.  The module then has the shard's `out_features` / `in_features`.
    """
    ckpt = Checkpoint(directory)
    if compression_config is None and max_memory_MB is not None:
        compression_config = retrieve_compression_config(ckpt.compression_configs(), max_memory_MB)
    if compression_config is None and niter is None:
        raise ValueError("one of compression_config, max_memory_MB or niter is needed")
    projections = discover_projections(ckpt)
    wanted = list(names) if names is not None else sorted(projections, key=lambda s: (int(s.split(".")[1]), s))
    dev = torch.device(device)
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world size {world}")
    if shard_rule is None:
        shard_rule = default_shard_rule
    out: Dict[str, BitStackLinear] = {}
    for lname in wanted:
        if lname not in projections:
            raise KeyError(f"{lname}: no such BitStack projection in {directory}")
        prefix = projections[lname]
        nb = int(compression_config[lname]) if compression_config is not None else int(niter)
        have = stored_blocks(ckpt, prefix)
        if nb < 0 or nb > have:
            raise ValueError(f"{lname}: {nb} blocks requested, the checkpoint stores {have}")
        _, u_shape = ckpt.info(f"{prefix}.u_0")
        _, vt_shape = ckpt.info(f"{prefix}.vt_0")
        out_features, kk = u_shape
        in_features = vt_shape[1]
        if kk != k or vt_shape[0] != k:
            raise ValueError(f"{lname}: checkpoint rank is {kk}, k={k} was asked for")
        has_bias = f"{prefix}.bias" in ckpt
        kind = shard_rule(lname) if world > 1 else None
        if kind not in (None, "rows", "cols"):
            raise ValueError(f"{lname}: shard rule returned {kind!r}")
        full_out, full_in = out_features, in_features
        if kind == "rows":
            if full_out % world or (full_out // world * full_in) % 8:
                raise ValueError(f"{lname}: {full_out} output rows cannot be cut into {world} byte-aligned shards")
            out_features = full_out // world
        elif kind == "cols":
            if full_in % (8 * world):
                raise ValueError(f"{lname}: {full_in} input columns cannot be cut into {world} byte-aligned shards")
            in_features = full_in // world
        # a column shard's outputs are partial sums: only rank 0 adds the bias, so that the all-reduce adds it once
        keep_bias = has_bias and (kind != "cols" or rank == 0)
        mod = BitStackLinear(w_bit=0, in_features=in_features, out_features=out_features, k=k, bias=keep_bias,
                             no_avd=False, dev=dev, fused_level=fused_level)
        mod.name = lname
        q = torch.empty(nb, out_features * in_features // 8, dtype=torch.uint8, device=dev)
        u = torch.empty(nb, out_features, k, dtype=torch.float16, device=dev)
        vt = torch.empty(nb, k, in_features, dtype=torch.float16, device=dev)
        r0 = rank * out_features
        for j in range(nb):
            if kind == "rows":
                # rows [r0, r0 + out) of the sign matrix are one byte range of the flat qweight_j
                row_bytes = full_in // 8
                ckpt.read_rows_into(f"{prefix}.qweight_{j}", r0 * row_bytes, (r0 + out_features) * row_bytes, q[j])
                ckpt.read_rows_into(f"{prefix}.u_{j}", r0, r0 + out_features, u[j])
                ckpt.read_into(f"{prefix}.vt_{j}", vt[j])
            elif kind == "cols":
                hq = torch.empty(1, full_out * full_in // 8, dtype=torch.uint8)
                hu = torch.empty(1, full_out, k, dtype=torch.float16)
                hvt = torch.empty(1, k, full_in, dtype=torch.float16)
                ckpt.read_into(f"{prefix}.qweight_{j}", hq[0])
                ckpt.read_into(f"{prefix}.u_{j}", hu[0])
                ckpt.read_into(f"{prefix}.vt_{j}", hvt[0])
                sq, su, svt = sharding.shard_cols(hq, hu, hvt, full_out, full_in, rank, world)
                q[j].copy_(sq[0]); u[j].copy_(su[0]); vt[j].copy_(svt[0])
            else:
                ckpt.read_into(f"{prefix}.qweight_{j}", q[j])
                ckpt.read_into(f"{prefix}.u_{j}", u[j])
                ckpt.read_into(f"{prefix}.vt_{j}", vt[j])
        if keep_bias:
            if kind == "rows":
                ckpt.read_rows_into(f"{prefix}.bias", r0, r0 + out_features, mod.bias)
            else:
                ckpt.read_into(f"{prefix}.bias", mod.bias)
        mod.qweight, mod.u, mod.vt = q, u, vt
        mod.w_bit = nb
        mod._stacked_blocks = nb
        out[lname] = mod
    return out


def default_shard_rule(name: str) -> str:
    """Tensor-parallel cut of a decoder layer's projections: the two projections that consume a sharded activation
    (attention output, MLP down) are cut by input columns, all others by output rows."""
    return "cols" if name.endswith(("o_proj", "down_proj")) else "rows"


def checkpoint_budget_table(directory: str, k: int = 16) -> Dict[str, int]:
    """{`layer.{i}.{sub}`: bytes of one block} for a checkpoint: the `memory_per_bit` table that
    `generate_configs` consumes (main.py:176-180 builds it from the live modules)."""
    ckpt = Checkpoint(directory)
    table = {}
    for lname, prefix in discover_projections(ckpt).items():
        _, (out_features, _) = ckpt.info(f"{prefix}.u_0")
        _, (_, in_features) = ckpt.info(f"{prefix}.vt_0")
        table[lname] = memory_per_block(out_features, in_features, k)
    return table
