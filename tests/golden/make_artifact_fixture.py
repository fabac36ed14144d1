#!/usr/bin/env python3
"""Write tests/golden/artifacts_small/ (a tiny artifact directory in the reference's
on-disk format, packed with the reference's OWN idxN packer) and
tests/golden/artifact_vectors.npz (what the reference's OWN loader makes of it: the
fields of every loaded module and its reference-route forward on seeded inputs).

Run where a checkout of pkhairkh/rag-cache-engineering-qwen35-9b-flute is available:
    python tests/golden/make_artifact_fixture.py --reference <checkout>
Both outputs are committed; the tests only read them.

The skeleton the artifacts are swapped into (tests/helpers.py: tiny_skeleton) has one
decoder layer: linear_attn.in_proj_qkv (Linear 128 -> 384 with bias), mlp.gate_proj /
up_proj (128 -> 256), mlp.down_proj (256 -> 128) and post_attention_layernorm.weight [128].
Coverage: fused QKV components (4-bit, gs 64, one component with a second 2-bit stream),
rotation + AWQ compensation recovered from a norm-gain edit (gate/up), a 3-bit tensor,
a low-rank residual and a stale recorded group_size (down).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def sha(path):
    return hashlib.sha256(open(path, "rb").read()).hexdigest()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its own Python modules are imported from it)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src", "scripts"))
    sys.path.insert(0, os.path.join(args.reference, "src", "flute_extended"))
    import palettized_modules as pm
    from make_golden import _store
    from helpers_skeleton import tiny_skeleton
    idxn = pm._get_idxn()
    torch.set_num_threads(1)
    out_dir = os.path.join(HERE, "artifacts_small")
    shutil.rmtree(out_dir, ignore_errors=True)
    os.makedirs(os.path.join(out_dir, "norm_edits"))
    rng = np.random.default_rng(2024)
    g = torch.Generator().manual_seed(2024)

    def stream(stem, N, K, bits, gs, tag="", scale=0.02):
        idx = rng.integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
        name = f"{stem}.idx{bits}{tag}"
        lname = f"{stem}.lut_scalar{tag}"
        idxn.pack_idxn(idx, bits).tofile(os.path.join(out_dir, name))
        lut = (scale * torch.randn(-(-N // gs), 1 << bits, generator=g)).sort(dim=1).values.half()
        lut.numpy().tofile(os.path.join(out_dir, lname))
        return name, lname

    def meta_for(stem, N, K, bits, gs, shape=True, recorded_gs=None):
        name, lname = stream(stem, N, K, bits, gs)
        m = {"index_file": name, "lut_file": lname, "bitwidth": bits,
             "group_size": gs if recorded_gs is None else recorded_gs,
             "indices_layout": f"idx{bits}", "sha256_idx": sha(os.path.join(out_dir, name)),
             "sha256_lut": sha(os.path.join(out_dir, lname)),
             "packed_len_bytes": N * K * bits // 8}
        if shape:
            m["dense_shape"] = [N, K]
        return m

    def add_stream2(m, stem, N, K, bits2, gs):
        name2, lname2 = stream(stem, N, K, bits2, gs, tag=".2", scale=0.005)
        m["streams"] = [{"file": m["index_file"]},
                        {"file": name2, "sha256": sha(os.path.join(out_dir, name2)),
                         "sha256_lut": sha(os.path.join(out_dir, lname2)),
                         "n_groups": -(-N // gs), "gs": gs, "bitwidth": bits2}]

    tensors = {}
    K = 128
    qkv = {"var": "model.layers.0.linear_attn.in_proj_qkv.weight", "dense_shape": [384, K],
           "components": {}}
    for key in ("Q", "K", "V"):
        cm = meta_for(f"l0_qkv_{key}", 128, K, 4, 64, shape=False)
        if key == "V":
            add_stream2(cm, f"l0_qkv_{key}", 128, K, 2, 64)
        qkv["components"][key] = cm
    tensors[qkv["var"]] = qkv

    # AWQ scale folded into the norm gain; gate/up are rotated and consume that norm
    s = (0.6 + 0.4 * torch.rand(K, generator=g)).float()
    edited = ((1.0 + torch.zeros(K)) / s - 1.0).numpy().astype(np.float32)
    np.save(os.path.join(out_dir, "norm_edits", "l0_post_norm.npy"), edited)
    s_rec = 1.0 / (1.0 + torch.from_numpy(edited))
    awq_stats = {"applied": True, "fold_order": "rotate_then_awq", "s_min": float(s_rec.min()),
                 "s_max": float(s_rec.max()), "s_mean": float(s_rec.mean())}
    for leaf, bits in (("gate_proj", 4), ("up_proj", 3)):
        m = meta_for(f"l0_mlp_{leaf}", 256, K, bits, 128)
        m["var"] = f"model.layers.0.mlp.{leaf}.weight"
        m["rotation"] = {"seed": 5, "k": K}
        m["awq"] = dict(awq_stats)
        tensors[m["var"]] = m
    norm_doc = {"edits": {"model.layers.0.post_attention_layernorm.weight": {
        "file": "norm_edits/l0_post_norm.npy",
        "sha256": sha(os.path.join(out_dir, "norm_edits", "l0_post_norm.npy")), "alpha": 0.5,
        "consumers": ["model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.up_proj.weight"]}}}
    json.dump(norm_doc, open(os.path.join(out_dir, "norm_gain_edits.json"), "w"), indent=1)

    down = meta_for("l0_mlp_down_proj", 128, 256, 4, 32, recorded_gs=31)   # stale recorded gs
    down["var"] = "model.layers.0.mlp.down_proj.weight"
    rank = 4
    (0.05 * torch.randn(128, rank, generator=g)).half().numpy().tofile(os.path.join(out_dir, "l0_mlp_down_proj.resA"))
    (0.05 * torch.randn(rank, 256, generator=g)).half().numpy().tofile(os.path.join(out_dir, "l0_mlp_down_proj.resB"))
    down["residual"] = {"resA_file": "l0_mlp_down_proj.resA", "resB_file": "l0_mlp_down_proj.resB",
                        "rank": rank, "sha256_resA": sha(os.path.join(out_dir, "l0_mlp_down_proj.resA")),
                        "sha256_resB": sha(os.path.join(out_dir, "l0_mlp_down_proj.resB"))}
    tensors[down["var"]] = down
    json.dump({"tensors": tensors}, open(os.path.join(out_dir, "metadata.json"), "w"), indent=1)

    # ---- what the reference's loader makes of it -------------------------------------------
    model = tiny_skeleton().half()
    metadata = pm.load_metadata(out_dir)
    scales = pm._recover_awq_scales(model, out_dir, metadata, pm._read_norm_gain_doc(out_dir))
    pm.apply_norm_gain_edits(model, out_dir)
    pm.replace_linear_with_palettized(model, metadata, out_dir, residual=True, reference=True,
                                      awq_scales=scales)
    out = {}
    layer = model.model.layers[0]
    _store(out, "norm_after_edit", layer.post_attention_layernorm.weight.data)
    out["fused_mlp_class"] = np.array([type(layer.mlp).__name__ == "FusedPalettizedMLP"])
    mods = {"q": layer.linear_attn.in_proj_qkv.q_proj, "k": layer.linear_attn.in_proj_qkv.k_proj,
            "v": layer.linear_attn.in_proj_qkv.v_proj, "gate": layer.mlp.gate_proj,
            "up": layer.mlp.up_proj, "down": layer.mlp.down_proj}
    for tag, m in mods.items():
        out[tag + "_meta"] = np.array([m.N, m.K, m.group_size, m.bitwidth,
                                       m.bitwidth2 if m.indices2 is not None else -1,
                                       -1 if m.resA is None else m.resA.shape[1]], dtype=np.int64)
        out[tag + "_blob_sha"] = np.frombuffer(hashlib.sha256(m.indices.numpy().tobytes()).digest(), dtype=np.uint8).copy()
        _store(out, tag + "_lut", m.lut.data)
        if m.bias is not None:
            _store(out, tag + "_bias", m.bias.data)
        if getattr(m, "awq_scale", None) is not None:
            _store(out, tag + "_awq", m.awq_scale.float())
        x = torch.randn(3, m.K, generator=g).half()
        with torch.no_grad():
            y = m(x)
        _store(out, tag + "_x", x)
        _store(out, tag + "_y", y)
    x = torch.randn(2, K, generator=g).half()
    with torch.no_grad():
        _store(out, "qkv_x", x)
        _store(out, "qkv_y", layer.linear_attn.in_proj_qkv(x))
        _store(out, "mlp_x", x)
        _store(out, "mlp_y", layer.mlp(x))
    path = os.path.join(HERE, "artifact_vectors.npz")
    np.savez_compressed(path, **out)
    total = sum(os.path.getsize(os.path.join(dp, f)) for dp, _, fs in os.walk(out_dir) for f in fs)
    print(f"wrote {out_dir} ({total} bytes) and {path} ({os.path.getsize(path)} bytes, {len(out)} arrays)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
