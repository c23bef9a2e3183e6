"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own Python modules unchanged (CPU only), feeds them
seeded inputs and stores inputs + outputs as .npz files.  The tests then read
only the .npz files, so they run where the reference is absent.

What each fixture pins (reference symbol -> file):
  pack_kat.npz        pack_sign / unpack_sign on ragged and aligned shapes
                      (bitstack/utils/pack_utils.py:5-26)
  decomp_small.npz    BitStackLinear.from_linear + forward_l0, 64x96, 4 blocks,
                      with bias (bitstack/modules/BitStackLinear.py:49-114)
  decomp_1024.npz     the "real weights" configuration scaled to 1024x1024:
                      W~N(0,0.02), niter 8, k 16, y at 2/4/8 blocks
  synth_l0.npz        forward_l0 outputs for seeded synthetic layers whose
                      inputs are regenerated from the seed (oracle.synthetic_layer)
  budget.json         retrieve_compression_config / generate_configs
                      (bitstack/utils/model_utils.py:53-66,179-187)
"""
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _import_reference(ref_root):
    sys.path.insert(0, ref_root)
    from bitstack.modules.BitStackLinear import BitStackLinear
    from bitstack.utils import pack_utils
    # model_utils imports plotting / dispatch packages that are not installed, so
    # the module cannot be imported; the two pure functions we need are compiled
    # from its source text, unchanged, instead.
    import ast
    path = os.path.join(ref_root, "bitstack", "utils", "model_utils.py")
    tree = ast.parse(open(path).read())
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef)
              and n.name in ("retrieve_compression_config", "generate_configs")]
    model_utils = types.SimpleNamespace()
    ns = {}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), path, "exec"), ns)
    model_utils.retrieve_compression_config = ns["retrieve_compression_config"]
    model_utils.generate_configs = ns["generate_configs"]
    return BitStackLinear, pack_utils, model_utils


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    ref_root = sys.argv[1]
    BitStackLinear, pack_utils, model_utils = _import_reference(ref_root)
    sys.path.insert(0, ROOT)
    from oracle import bitstack_oracle as orc

    torch.manual_seed(1234)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- pack / unpack ------------------------------------------------------
    out = {}
    kat = torch.tensor([1] + [-1] * 7 + [-1] * 7 + [1], dtype=torch.int8)
    out["kat_sign"] = kat.numpy()
    out["kat_packed"] = pack_utils.pack_sign(kat).numpy()
    shapes = [(1, 8), (3, 5), (7, 9), (16, 24), (5, 64), (33, 130), (128, 256)]
    g = torch.Generator().manual_seed(7)
    for i, shp in enumerate(shapes):
        s = (torch.randint(0, 2, shp, generator=g, dtype=torch.int8) * 2 - 1)
        p = pack_utils.pack_sign(s)
        r = pack_utils.unpack_sign(p, torch.Size(shp))
        r2 = pack_utils.unpack_sign_v2(p, torch.Size(shp))
        assert r.equal(s) and r2.equal(s)
        out[f"sign_{i}"] = s.numpy()
        out[f"packed_{i}"] = p.numpy()
    out["n_cases"] = np.array(len(shapes))
    np.savez_compressed(os.path.join(HERE, "pack_kat.npz"), **out)

    # ---- real decompositions ------------------------------------------------
    def decomp_case(m, n, niter, bias, rows_list, bits_list, seed, fname, std=0.02):
        torch.manual_seed(seed)
        lin = torch.nn.Linear(n, m, bias=bias)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(m, n) * std)
            if bias:
                lin.bias.copy_(torch.randn(m) * 0.1)
        if bias:  # the reference flow converts a model to fp16 first; keeps bias fp16
            lin = lin.half()
        w0 = lin.weight.detach().float().clone()
        with torch.no_grad():  # the reference decomposes under torch.no_grad (utils/decompose.py:7)
            q = BitStackLinear.from_linear(lin, w_bit=niter, k=16, bias=bias)
        d = {
            "weight": w0.numpy() if m * n <= 64 * 96 else np.zeros(0, np.float32),
            "qweight": np.stack([getattr(q, f"qweight_{i}").numpy() for i in range(niter)]),
            "u": np.stack([getattr(q, f"u_{i}").numpy() for i in range(niter)]),
            "vt": np.stack([getattr(q, f"vt_{i}").numpy() for i in range(niter)]),
            "bits": np.array(bits_list),
            "rows": np.array(rows_list),
            "seed": np.array(seed),
        }
        if bias:
            d["bias"] = q.bias.detach().numpy().astype(np.float16)
        for rows in rows_list:
            x = torch.randn(rows, n).half()
            d[f"x_{rows}"] = x.numpy()
            for b in bits_list:
                q.set_bit(b)
                d[f"y_{rows}_{b}"] = q.forward(x).numpy()
        q.set_bit(niter)
        np.savez_compressed(os.path.join(HERE, fname), **d)
        return d

    decomp_case(64, 96, 4, True, [1, 3], [1, 2, 4], 11, "decomp_small.npz")
    decomp_case(1024, 1024, 8, False, [1, 4], [2, 4, 8], 12, "decomp_1024.npz")

    # ---- synthetic layers: only outputs are stored --------------------------
    syn = {}
    cases = [  # (M, N, blocks_total, seed, rows, active)
        (1024, 4096, 16, 101, 1, (2, 8, 16)),
        (1024, 4096, 16, 101, 4, (5,)),
        (256, 512, 6, 102, 16, (1, 6)),
        (4096, 1024, 4, 103, 1, (3,)),
    ]
    meta = []
    for (m, n, nb, seed, rows, actives) in cases:
        qw, u, vt = orc.synthetic_layer(m, n, nb, seed)
        x = orc.synthetic_input(rows, n, seed + 1000)
        mod = BitStackLinear(w_bit=nb, in_features=n, out_features=m, k=16, bias=False, no_avd=False, dev="cpu")
        for j in range(nb):
            setattr(mod, f"qweight_{j}", torch.from_numpy(qw[j]))
            setattr(mod, f"u_{j}", torch.from_numpy(u[j]))
            setattr(mod, f"vt_{j}", torch.from_numpy(vt[j]))
        for a in actives:
            mod.set_bit(a)
            y = mod.forward(torch.from_numpy(x))
            syn[f"y_{m}_{n}_{seed}_{rows}_{a}"] = y.numpy()
            meta.append([m, n, nb, seed, rows, a])
    syn["cases"] = np.array(meta)
    np.savez_compressed(os.path.join(HERE, "synth_l0.npz"), **syn)

    # ---- budget arithmetic ----------------------------------------------------
    if model_utils is not None:
        mem = {"layer.0.self_attn.q_proj": 2359296, "layer.0.self_attn.k_proj": 688128,
               "layer.0.mlp.down_proj": 7929856}
        order = ["layer.0.mlp.down_proj", "layer.0.self_attn.q_proj", "layer.0.self_attn.k_proj",
                 "layer.0.self_attn.q_proj", "layer.0.mlp.down_proj", "layer.0.self_attn.k_proj"]
        total = sum(mem.values()) + 123456
        cfgs = model_utils.generate_configs(order, mem, total)
        picks = {}
        for mb in (10.6, 11, 13, 20, 25, 100):
            picks[str(mb)] = model_utils.retrieve_compression_config(cfgs, mb)
        try:
            model_utils.retrieve_compression_config(cfgs, 1)
            too_small = "no error"
        except ValueError as e:
            too_small = str(e)
        with open(os.path.join(HERE, "budget.json"), "w") as f:
            json.dump({"memory_per_bit": mem, "order": order, "total": total, "configs": cfgs,
                       "picks": picks, "too_small_error": too_small}, f, indent=1)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
