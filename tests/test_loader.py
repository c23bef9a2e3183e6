"""Budget selection and partial checkpoint loading (CPU): the loader against the reference-generated
budget fixture, against the `safetensors` package's own reader/writer, and against the bytes it must
pick out of a sharded checkpoint."""
import json
import os

import numpy as np
import pytest
import torch

from bitstack_b200 import loader
from oracle import bitstack_oracle as orc


def _fake_checkpoint(tmp_path, n_layers=2, blocks=4, shards=2, seed=0):
    shapes = {"self_attn.q_proj": (64, 128), "self_attn.k_proj": (16, 128), "mlp.down_proj": (128, 192)}
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for i in range(n_layers):
        for sub, (m, n) in shapes.items():
            p = f"model.layers.{i}.{sub}"
            for j in range(blocks):
                tensors[f"{p}.qweight_{j}"] = torch.randint(0, 256, (m * n // 8,), dtype=torch.uint8, generator=g)
                tensors[f"{p}.u_{j}"] = torch.randn(m, 16, generator=g).abs().half()
                tensors[f"{p}.vt_{j}"] = torch.randn(16, n, generator=g).abs().half()
        tensors[f"model.layers.{i}.input_layernorm.weight"] = torch.ones(128).half()
    tensors["model.layers.1.mlp.down_proj.bias"] = torch.randn(128, generator=g).half()
    names = sorted(tensors)
    weight_map = {}
    for s in range(shards):
        part = {k: tensors[k] for k in names[s::shards]}
        fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        loader.write_safetensors(os.path.join(tmp_path, fname), part, metadata={"format": "pt"})
        weight_map.update({k: fname for k in part})
    with open(os.path.join(tmp_path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    return tensors, shapes


def test_budget_functions_match_reference_fixture(golden_dir):
    with open(os.path.join(golden_dir, "budget.json")) as f:
        fx = json.load(f)
    configs = loader.generate_configs(fx["order"], fx["memory_per_bit"], fx["total"])
    assert configs == fx["configs"]
    for mb, layers in fx["picks"].items():
        assert loader.retrieve_compression_config(configs, float(mb)) == layers
    with pytest.raises(ValueError) as e:
        loader.retrieve_compression_config(configs, 1)
    assert str(e.value) == fx["too_small_error"]


def test_safetensors_reader_and_writer_agree_with_the_library(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    g = torch.Generator().manual_seed(3)
    tensors = {"a.qweight_0": torch.randint(0, 256, (77,), dtype=torch.uint8, generator=g),
               "a.u_0": torch.randn(5, 16, generator=g).half(), "b": torch.randn(3, 2, generator=g),
               "empty": torch.zeros(0, 4).half()}
    # their writer, our reader
    p1 = os.path.join(tmp_path, "theirs.safetensors")
    st.save_file(tensors, p1)
    f1 = loader.SafetensorsFile(p1)
    assert set(f1.keys()) == set(tensors)
    for k, t in tensors.items():
        assert torch.equal(f1.read(k), t)
    # our writer, their reader
    p2 = os.path.join(tmp_path, "ours.safetensors")
    loader.write_safetensors(p2, tensors, metadata={"format": "pt"})
    back = st.load_file(p2)
    assert set(back) == set(tensors)
    for k, t in tensors.items():
        assert torch.equal(back[k], t)


def test_truncated_or_inconsistent_files_are_rejected(tmp_path):
    p = os.path.join(tmp_path, "x.safetensors")
    loader.write_safetensors(p, {"t": torch.arange(16, dtype=torch.uint8)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-4])
    with pytest.raises(ValueError, match="inconsistent offsets"):
        loader.SafetensorsFile(p)
    open(p, "wb").write(raw[:5])
    with pytest.raises(ValueError, match="not a safetensors file"):
        loader.SafetensorsFile(p)


def test_partial_load_takes_exactly_the_budgeted_blocks(tmp_path):
    tensors, shapes = _fake_checkpoint(tmp_path)
    table = loader.checkpoint_budget_table(str(tmp_path))
    assert table["layer.0.self_attn.q_proj"] == orc.memory_per_block(64, 128) == 64 * 128 // 8 + 32 * (64 + 128)
    assert set(table) == {f"layer.{i}.{s}" for i in range(2) for s in shapes}
    # budget steps in a fixed order, then the biggest configuration under a limit
    order = [n for n in sorted(table) for _ in range(3)]
    extra = 12345
    configs = loader.generate_configs(order, table, sum(table.values()) + extra)
    with open(os.path.join(tmp_path, "compression_config.json"), "w") as f:
        json.dump(configs, f)
    limit_mb = configs[7]["memory"] / 1024 ** 2 + 1e-6
    mods = loader.load_bitstack_linears(str(tmp_path), max_memory_MB=limit_mb, device="cpu")
    chosen = configs[7]["layers"]
    assert {n: m.w_bit for n, m in mods.items()} == chosen
    assert sum(table[n] * (b - 1) for n, b in chosen.items()) + sum(table.values()) + extra == configs[7]["memory"]
    for lname, mod in mods.items():
        i, sub = lname.split(".", 2)[1:]
        p = f"model.layers.{i}.{sub}"
        nb = chosen[lname]
        assert mod.name == lname and mod._stacked_blocks == nb
        assert mod.qweight.shape == (nb, mod.out_features * mod.in_features // 8)
        for j in range(nb):
            assert torch.equal(mod.qweight[j], tensors[f"{p}.qweight_{j}"])
            assert torch.equal(mod.u[j], tensors[f"{p}.u_{j}"])
            assert torch.equal(mod.vt[j], tensors[f"{p}.vt_{j}"])
        if lname == "layer.1.mlp.down_proj":
            assert torch.equal(mod.bias, tensors[f"{p}.bias"])
        else:
            assert mod.bias is None


def test_loader_argument_errors(tmp_path):
    _fake_checkpoint(tmp_path, blocks=2)
    with pytest.raises(ValueError, match="one of compression_config"):
        loader.load_bitstack_linears(str(tmp_path), device="cpu")
    with pytest.raises(ValueError, match="the checkpoint stores 2"):
        loader.load_bitstack_linears(str(tmp_path), niter=3, device="cpu")
    with pytest.raises(KeyError):
        loader.load_bitstack_linears(str(tmp_path), niter=1, device="cpu", names=["layer.9.self_attn.q_proj"])
    mods = loader.load_bitstack_linears(str(tmp_path), niter=1, device="cpu", names=["layer.1.self_attn.k_proj"])
    assert list(mods) == ["layer.1.self_attn.k_proj"] and mods["layer.1.self_attn.k_proj"].w_bit == 1


@pytest.mark.gpu
def test_loaded_checkpoint_runs_on_the_gpu_path(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    q, u, vt = orc.synthetic_layer(256, 512, 3, seed=5)
    tensors = {}
    for j in range(3):
        tensors[f"model.layers.0.mlp.up_proj.qweight_{j}"] = torch.from_numpy(np.ascontiguousarray(q[j]))
        tensors[f"model.layers.0.mlp.up_proj.u_{j}"] = torch.from_numpy(np.ascontiguousarray(u[j]))
        tensors[f"model.layers.0.mlp.up_proj.vt_{j}"] = torch.from_numpy(np.ascontiguousarray(vt[j]))
    loader.write_safetensors(os.path.join(tmp_path, "model.safetensors"), tensors)
    mods = loader.load_bitstack_linears(str(tmp_path), {"layer.0.mlp.up_proj": 2}, device=dev)
    mod = mods["layer.0.mlp.up_proj"]
    for rows in (1, 9):
        x_np = orc.synthetic_input(rows, 512, seed=rows)
        y = mod(torch.from_numpy(x_np).to(dev)).float().cpu().numpy()
        ref = orc.forward_f64(x_np, q, u, vt, 2, None)
        assert orc.max_normalised_error(y, ref) <= 4e-3
    mod.set_bit(1)   # lowering the budget needs no reload
    x_np = orc.synthetic_input(1, 512, seed=77)
    y = mod(torch.from_numpy(x_np).to(dev)).float().cpu().numpy()
    assert orc.max_normalised_error(y, orc.forward_f64(x_np, q, u, vt, 1, None)) <= 4e-3


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_placement_reads_this_ranks_shard(tmp_path, world):
    """`rank` / `world`: every rank's modules hold exactly `sharding.shard_rows` / `shard_cols` of the full tensors,
    the row shards concatenate and the column-shard partial sums add up to the single-device float64 result, and a
    bias lives on rank 0 only for a column-sharded projection."""
    from bitstack_b200 import sharding
    tensors, shapes = _fake_checkpoint(tmp_path, n_layers=2, blocks=3, shards=2, seed=5)
    cfg = {f"layer.{i}.{sub}": 2 + (i + k) % 2 for i in range(2) for k, sub in enumerate(shapes)}
    full = loader.load_bitstack_linears(str(tmp_path), cfg, device="cpu")
    per_rank = [loader.load_bitstack_linears(str(tmp_path), cfg, device="cpu", rank=r, world=world) for r in range(world)]
    x_rng = np.random.default_rng(1)
    for name, mod in full.items():
        m, n = mod.out_features, mod.in_features
        nb = cfg[name]
        kind = loader.default_shard_rule(name)
        x = x_rng.standard_normal((2, n)).astype(np.float16)
        y_full = orc.forward_f64(x, mod.qweight.numpy(), mod.u.numpy(), mod.vt.numpy(), nb)
        acc = []
        for r in range(world):
            sm = per_rank[r][name]
            cut = sharding.shard_rows if kind == "rows" else sharding.shard_cols
            q, u, vt = cut(mod.qweight, mod.u, mod.vt, m, n, r, world)
            assert torch.equal(sm.qweight, q) and torch.equal(sm.u, u) and torch.equal(sm.vt, vt), (name, r)
            assert sm.w_bit == nb and sm.name == name
            if kind == "rows":
                assert (sm.out_features, sm.in_features) == (m // world, n)
                acc.append(orc.forward_f64(x, q.numpy(), u.numpy(), vt.numpy(), nb))
            else:
                assert (sm.out_features, sm.in_features) == (m, n // world)
                assert (sm.bias is not None) == (mod.bias is not None and r == 0)
                lo = r * (n // world)
                acc.append(orc.forward_f64(x[:, lo:lo + n // world], q.numpy(), u.numpy(), vt.numpy(), nb))
        y = np.concatenate(acc, axis=1) if kind == "rows" else np.sum(acc, axis=0)
        assert np.abs(y - y_full).max() <= 1e-9 * max(np.abs(y_full).max(), 1.0)
    with pytest.raises(ValueError):
        loader.load_bitstack_linears(str(tmp_path), cfg, device="cpu", rank=2, world=2)
    # 16 output rows of k_proj cannot be cut into 32 shards
    with pytest.raises(ValueError):
        loader.load_bitstack_linears(str(tmp_path), cfg, device="cpu", rank=0, world=32)
