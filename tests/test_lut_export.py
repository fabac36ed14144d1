"""The palette codec (export_luts / import_luts) against a directory the reference's own
codec wrote (tests/golden/pretrained_luts_small/, made by
tests/golden/make_lut_export_fixture.py; that script also verified that the reference's
strict import accepts what this repo's codec writes)."""
from __future__ import annotations

import importlib
import json
import os
import shutil

import numpy as np
import pytest
import torch

from helpers import TOL, pkg, rel_err
from helpers_skeleton import tiny_skeleton

HERE = os.path.dirname(os.path.abspath(__file__))
ART = os.path.join(HERE, "golden", "artifacts_small")
LUTS = os.path.join(HERE, "golden", "pretrained_luts_small")
codec = importlib.import_module(pkg.__name__ + ".lut_export")
loader = importlib.import_module(pkg.__name__ + ".loader")


@pytest.fixture(scope="module")
def vec():
    z = np.load(os.path.join(HERE, "golden", "lut_export_vectors.npz"))

    def get(key):
        if key + "__f16" in z:
            return torch.from_numpy(z[key + "__f16"].view(np.int16).copy()).view(torch.float16)
        return torch.from_numpy(z[key]) if z[key].dtype.kind != "U" else z[key]
    get.has = lambda key: key in z or key + "__f16" in z
    return get


def _model(device="cpu"):
    return loader.load_quant_model(ART, tiny_skeleton, device, residual=True)[0]


def test_import_installs_the_reference_written_palettes(vec):
    model = _model()
    before = {n: m.lut.clone() for n, m in codec.iter_palettized_linears(model)}
    res = codec.import_luts(model, LUTS)
    names = [str(n) for n in vec("names")]
    assert sorted(res["loaded"]) == names and res["checked"] == 6 and not res["mismatches"]
    for name, m in codec.iter_palettized_linears(model):
        assert torch.equal(m.lut, vec(f"lut::{name}")) and not torch.equal(m.lut, before[name])
        assert m.lut.dtype == torch.float16
        if m.lut2 is not None:
            assert torch.equal(m.lut2, vec(f"lut2::{name}"))
    assert bool(vec("cross_import_ok")[0])


def test_export_reproduces_the_reference_digests_and_round_trips(tmp_path):
    model = _model()
    codec.import_luts(model, LUTS)
    ref_manifest = json.load(open(os.path.join(LUTS, "manifest.json")))
    mine = codec.export_luts(model, str(tmp_path / "out"), extra_meta={"source": "test"})
    assert mine["code_sha256"] == ref_manifest["code_sha256"]      # content digests are the reference's
    assert mine["files"] == ref_manifest["files"] and mine["n_modules"] == 6
    assert mine["version"] == ref_manifest["version"] == codec.LUT_EXPORT_VERSION
    with np.load(os.path.join(LUTS, "model__layers__0__mlp__gate_proj.npz")) as a, \
            np.load(str(tmp_path / "out" / "model__layers__0__mlp__gate_proj.npz")) as b:
        assert sorted(a.files) == sorted(b.files)
        for k in a.files:
            if k != "header":
                assert a[k].dtype == b[k].dtype and np.array_equal(a[k], b[k]), k
    fresh = _model()
    res = codec.import_luts(fresh, str(tmp_path / "out"))
    assert len(res["loaded"]) == 6
    for (n1, m1), (n2, m2) in zip(codec.iter_palettized_linears(model),
                                  codec.iter_palettized_linears(fresh)):
        assert n1 == n2 and torch.equal(m1.lut, m2.lut)


def test_refusals_of_the_codec(tmp_path):
    model = _model()
    with pytest.raises(ValueError, match="no manifest.json"):
        codec.import_luts(model, str(tmp_path))
    with pytest.raises(ValueError, match="no PalettizedLinear"):
        codec.export_luts(torch.nn.Linear(4, 4), str(tmp_path / "x"))
    with pytest.raises(TypeError):
        codec.export_luts(model, str(tmp_path / "x"), extra_meta=[1])
    with pytest.raises(ValueError, match="JSON-serializable"):
        codec.export_luts(model, str(tmp_path / "x"), extra_meta={"a": object()})
    bf = _model()
    gate = bf.model.layers[0].mlp.gate_proj
    gate.register_buffer("lut", gate.lut.bfloat16(), persistent=False)
    with pytest.raises(RuntimeError, match="fp16 deployment grid"):
        codec.export_luts(bf, str(tmp_path / "x"))
    # a file changed after export
    d = str(tmp_path / "a")
    shutil.copytree(LUTS, d)
    with open(os.path.join(d, "model__layers__0__mlp__down_proj.npz"), "r+b") as f:
        f.seek(200)
        f.write(b"\x01\x02\x03")
    with pytest.raises(ValueError, match="sha256 mismatch"):
        codec.import_luts(_model(), d)
    res = codec.import_luts(_model(), d, strict=False)
    assert len(res["loaded"]) == 5 and len(res["mismatches"]) == 1
    # geometry drift: the live module has another group size
    drift = _model()
    drift.model.layers[0].mlp.down_proj.group_size = 64
    with pytest.raises(ValueError, match="geometry"):
        codec.import_luts(drift, LUTS)
    # coverage drift in both directions
    d = str(tmp_path / "b")
    shutil.copytree(LUTS, d)
    man = json.load(open(os.path.join(d, "manifest.json")))
    gone = man["files"].pop("model.layers.0.mlp.up_proj")
    json.dump(man, open(os.path.join(d, "manifest.json"), "w"))
    with pytest.raises(ValueError, match="not covered by the manifest"):
        codec.import_luts(_model(), d)
    man["files"]["model.layers.9.mlp.up_proj"] = gone
    json.dump(man, open(os.path.join(d, "manifest.json"), "w"))
    with pytest.raises(ValueError, match="no live PalettizedLinear"):
        codec.import_luts(_model(), d)
    man["version"] = 2
    json.dump(man, open(os.path.join(d, "manifest.json"), "w"))
    with pytest.raises(ValueError, match="manifest version"):
        codec.import_luts(_model(), d)


@pytest.mark.gpu
def test_kernels_serve_the_imported_palettes(vec):
    model = _model("cuda")
    layer = model.model.layers[0]
    v, down = layer.linear_attn.in_proj_qkv.v_proj, layer.mlp.down_proj
    old = down(vec("down_x").cuda()).float().cpu()
    codec.import_luts(model, LUTS)
    assert down.lut.is_cuda
    for tag, m in (("v", v), ("down", down)):
        y = m(vec(tag + "_x").cuda())
        assert rel_err(y.float().cpu(), vec(tag + "_y").float()) <= TOL, tag
    assert rel_err(old, vec("down_y").float()) > TOL      # the palettes did move the output
