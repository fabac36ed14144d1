#!/usr/bin/env python3
"""Write two tiny head-artifact directories in the reference's on-disk format (packed with
the reference's OWN idxN packer) and tests/golden/heads_vectors.npz (what the reference's
OWN swap makes of them, used as `heads_dir` beside tests/golden/artifacts_small/):

  artifacts_heads_tied/    one set under the lm_head name carrying "tied": true — 4-bit codes
                           plus a 4-bit second stream (the reference's tied-pair entry builds
                           the embedding consumer at the first stream's width), rank-4 residual,
                           rotation record; the embedding consumer shares it and un-rotates
                           its rows
  artifacts_heads_untied/  lm_head (4-bit, rotated) and embed_tokens (3-bit, rank-4 residual,
                           not rotated) as separate sets

Run where a checkout of pkhairkh/rag-cache-engineering-qwen35-9b-flute is available:
    python tests/golden/make_heads_fixture.py --reference <checkout>
All outputs are committed; the tests only read them.
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
VOCAB, HIDDEN = 256, 128


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
    from helpers_skeleton import tiny_skeleton_with_heads
    idxn = pm._get_idxn()
    torch.set_num_threads(1)
    rng = np.random.default_rng(77)
    g = torch.Generator().manual_seed(77)

    def write_set(out_dir, stem, var, bits, gs, bits2=None, rank=0, rot=None, tied=False):
        def stream(b, tag="", scale=0.02):
            idx = rng.integers(0, 1 << b, size=(VOCAB, HIDDEN), dtype=np.uint8)
            name, lname = f"{stem}.idx{b}{tag}", f"{stem}.lut_scalar{tag}"
            idxn.pack_idxn(idx, b).tofile(os.path.join(out_dir, name))
            (scale * torch.randn(-(-VOCAB // gs), 1 << b, generator=g)).half().numpy().tofile(
                os.path.join(out_dir, lname))
            return name, lname
        name, lname = stream(bits)
        m = {"var": var, "index_file": name, "lut_file": lname, "bitwidth": bits, "group_size": gs,
             "indices_layout": f"idx{bits}", "sha256_idx": sha(os.path.join(out_dir, name)),
             "sha256_lut": sha(os.path.join(out_dir, lname)),
             "packed_len_bytes": VOCAB * HIDDEN * bits // 8, "dense_shape": [VOCAB, HIDDEN]}
        if bits2:
            name2, lname2 = stream(bits2, tag=".2", scale=0.005)
            m["streams"] = [{"file": name},
                            {"file": name2, "sha256": sha(os.path.join(out_dir, name2)),
                             "sha256_lut": sha(os.path.join(out_dir, lname2)),
                             "n_groups": -(-VOCAB // gs), "gs": gs, "bitwidth": bits2}]
        if rank:
            for leaf, shape in (("resA", (VOCAB, rank)), ("resB", (rank, HIDDEN))):
                (0.05 * torch.randn(*shape, generator=g)).half().numpy().tofile(
                    os.path.join(out_dir, f"{stem}.{leaf}"))
            m["residual"] = {"resA_file": f"{stem}.resA", "resB_file": f"{stem}.resB", "rank": rank,
                             "sha256_resA": sha(os.path.join(out_dir, f"{stem}.resA")),
                             "sha256_resB": sha(os.path.join(out_dir, f"{stem}.resB"))}
        if rot is not None:
            m["rotation"] = {"seed": rot, "k": HIDDEN}
        if tied:
            m["tied"] = True
        return m

    out = {}
    ids = torch.from_numpy(rng.integers(0, VOCAB, size=(2, 5), dtype=np.int64))
    ids[0, 0], ids[1, 4] = VOCAB - 1, 0
    x = torch.randn(3, HIDDEN, generator=g).half()
    _store(out, "ids", ids)
    _store(out, "x", x)
    base = os.path.join(HERE, "artifacts_small")
    for variant in ("tied", "untied"):
        out_dir = os.path.join(HERE, f"artifacts_heads_{variant}")
        shutil.rmtree(out_dir, ignore_errors=True)
        os.makedirs(out_dir)
        if variant == "tied":
            tensors = {"model.lm_head.weight": write_set(out_dir, "lm_head", "model.lm_head.weight", 4,
                                                         64, bits2=4, rank=4, rot=3, tied=True)}
        else:
            tensors = {"model.lm_head.weight": write_set(out_dir, "lm_head", "model.lm_head.weight", 4,
                                                         128, rot=8),
                       "model.embed_tokens.weight": write_set(out_dir, "embed_tokens",
                                                              "model.embed_tokens.weight", 3, 64,
                                                              rank=4)}
        json.dump({"tensors": tensors}, open(os.path.join(out_dir, "metadata.json"), "w"), indent=1)

        model = tiny_skeleton_with_heads(HIDDEN, 256, VOCAB).half()
        metadata = pm.load_metadata(base)
        scales = pm._recover_awq_scales(model, base, metadata, pm._read_norm_gain_doc(base))
        pm.apply_norm_gain_edits(model, base)
        pm.replace_linear_with_palettized(model, metadata, base, residual=True, reference=True,
                                          awq_scales=scales, heads_dir=out_dir)
        lm, emb = model.lm_head, model.model.embed_tokens
        assert type(lm).__name__ == "PalettizedLinear" and type(emb).__name__ == "PalettizedEmbedding"
        if variant == "tied":
            assert emb.indices.data_ptr() == lm.indices.data_ptr()
        for tag, m in (("lm", lm), ("emb", emb)):
            out[f"{variant}_{tag}_meta"] = np.array(
                [m.N, m.K, m.group_size, m.bitwidth, m.bitwidth2 if m.indices2 is not None else -1,
                 -1 if m.resA is None else m.resA.shape[1],
                 -1 if m.rotation_seed is None else m.rotation_seed], dtype=np.int64)
            out[f"{variant}_{tag}_blob_sha"] = np.frombuffer(
                hashlib.sha256(m.indices.numpy().tobytes()).digest(), dtype=np.uint8).copy()
        with torch.no_grad():
            _store(out, f"{variant}_emb_y", emb(ids))
            _store(out, f"{variant}_lm_y", lm(x))
    path = os.path.join(HERE, "heads_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote the two head directories and {path} ({os.path.getsize(path)} bytes, {len(out)} arrays)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
