#!/usr/bin/env python3
"""Write tests/golden/pretrained_luts_small/ with the reference's OWN palette codec
(src/rag/lut_export.py: export_luts) and tests/golden/lut_export_vectors.npz.

The model is tests/golden/artifacts_small/ loaded by the reference's own loader; every
palette is then moved (scaled and shifted, re-snapped to float16, as a fine-tune would
leave it) and exported. The vectors hold the moved palettes and the reference-route forward
of two modules after the move. The script also checks the opposite direction on the spot: a
directory written by THIS repo's codec for the same model state is accepted by the
reference's strict import_luts and yields the same content digests.

Run where a checkout of pkhairkh/rag-cache-engineering-qwen35-9b-flute is available:
    python tests/golden/make_lut_export_fixture.py --reference <checkout>
Both outputs are committed; the tests only read them.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import shutil
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its own Python modules are imported from it)")
    args = ap.parse_args()
    for sub in ("scripts", "flute_extended", "rag"):
        sys.path.insert(0, os.path.join(args.reference, "src", sub))
    import palettized_modules as pm
    import lut_export as ref_codec
    from make_golden import _store
    from helpers_skeleton import tiny_skeleton
    torch.set_num_threads(1)
    base = os.path.join(HERE, "artifacts_small")
    out_dir = os.path.join(HERE, "pretrained_luts_small")
    shutil.rmtree(out_dir, ignore_errors=True)

    def load_reference_model():
        model = tiny_skeleton().half()
        metadata = pm.load_metadata(base)
        scales = pm._recover_awq_scales(model, base, metadata, pm._read_norm_gain_doc(base))
        pm.apply_norm_gain_edits(model, base)
        pm.replace_linear_with_palettized(model, metadata, base, residual=True, reference=True,
                                          awq_scales=scales)
        return model

    model = load_reference_model()
    out = {}
    g = torch.Generator().manual_seed(31)
    for i, (name, m) in enumerate(pm.iter_palettized_linears(model)):
        m.register_buffer("lut", (m.lut.float() * (1.1 + 0.05 * i) + 0.001).half(), persistent=False)
        if m.lut2 is not None:
            m.register_buffer("lut2", (m.lut2.float() * 0.9).half(), persistent=False)
        _store(out, f"lut::{name}", m.lut)
        if m.lut2 is not None:
            _store(out, f"lut2::{name}", m.lut2)
    manifest = ref_codec.export_luts(model, out_dir, extra_meta={"source": "fixture"})
    layer = model.model.layers[0]
    for tag, m in (("v", layer.linear_attn.in_proj_qkv.v_proj), ("down", layer.mlp.down_proj)):
        x = torch.randn(3, m.K, generator=g).half()
        with torch.no_grad():
            _store(out, tag + "_x", x)
            _store(out, tag + "_y", m(x))
    out["names"] = np.array(sorted(manifest["files"]))

    # the opposite direction: this repo's codec writes, the reference's strict import reads
    pkg = importlib.import_module("rag-cache-engineering-qwen35-9b-flute_b200")
    mine = importlib.import_module(pkg.__name__ + ".lut_export")
    loader = importlib.import_module(pkg.__name__ + ".loader")
    my_model, _ = loader.load_quant_model(base, tiny_skeleton, "cpu", residual=True)
    mine.import_luts(my_model, out_dir)
    with tempfile.TemporaryDirectory() as tmp:
        my_manifest = mine.export_luts(my_model, tmp, extra_meta={"source": "fixture"})
        assert my_manifest["code_sha256"] == manifest["code_sha256"]
        fresh = load_reference_model()
        res = ref_codec.import_luts(fresh, tmp, strict=True)
        assert sorted(res["loaded"]) == sorted(manifest["files"]) and not res["mismatches"]
        for name, m in pm.iter_palettized_linears(fresh):
            key = f"lut::{name}__f16"
            assert np.array_equal(m.lut.view(torch.int16).numpy().view(np.uint16), out[key])
    out["cross_import_ok"] = np.array([True])
    path = os.path.join(HERE, "lut_export_vectors.npz")
    np.savez_compressed(path, **out)
    total = sum(os.path.getsize(os.path.join(out_dir, f)) for f in os.listdir(out_dir))
    print(f"wrote {out_dir} ({total} bytes, {len(manifest['files'])} modules) and {path}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
