"""`load_quant_model` — the one entry that turns a model skeleton plus an artifact
directory into a model whose Linear layers run on the B200 LUT kernels.

Mirrors the reference's loader (src/scripts/loader.py:17-66 and
load_palettized_model, src/scripts/palettized_modules.py:3264-3398): metadata →
(pristine model) recover AWQ scales → apply norm-gain edits → swap modules →
fuse MLPs → move to the device. `forward="kernel"` serves through
libb200lut.so; `forward="reference"` keeps every module on the torch dequant
route (on CUDA that is this package's dequant kernel + a torch matmul).

Same positional arguments and defaults as the reference. `model_name` may also be an
`nn.Module` (any module tree with `model.layers[i].<path>` Linear members) or a
zero-argument callable that builds one; a string is handed to
`transformers.AutoModelForCausalLM.from_pretrained` (needs a local checkpoint).
The reference's vendored Qwen3.5 classes and their M1/M2 memories are model code
outside the linear path: the default `use_m1m2=True` without a gates file leaves
outputs unchanged in the reference and is served without the memories; a gates
file is refused.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import numpy as np
import torch

from . import artifacts

__all__ = ["load_quant_model", "apply_norm_gain_edits", "recover_awq_scales"]


def _norm_doc(artifacts_dir: str) -> Optional[Dict]:
    path = os.path.join(artifacts_dir, "norm_gain_edits.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)


def apply_norm_gain_edits(model, artifacts_dir: str, verify_sha: bool = True,
                          strict: bool = True) -> Dict:
    """Copy every edited RMSNorm gain (`norm_edits/*.npy`, complete parameters) into
    the named parameter. Idempotent. Follows palettized_modules.py:3029-3076."""
    doc = _norm_doc(artifacts_dir)
    if not doc:
        return {}
    art = artifacts.ArtifactDir(artifacts_dir, verify_sha)
    named = dict(model.named_parameters())
    applied = {}
    for pname, entry in (doc.get("edits") or {}).items():
        if pname not in named:
            if strict:
                raise KeyError(f"apply_norm_gain_edits: parameter {pname!r} not found in model")
            print(f"  WARNING: norm edit for unknown parameter {pname!r} skipped", flush=True)
            continue
        art.check_sha(entry["file"], entry.get("sha256"), f"norm_edit:{pname}")
        arr = np.load(art.file(entry["file"]))
        param = named[pname]
        if tuple(arr.shape) != tuple(param.shape):
            raise ValueError(f"norm_edit:{pname}: shape {arr.shape} != parameter shape "
                             f"{tuple(param.shape)}")
        param.data.copy_(torch.from_numpy(arr).to(param.dtype))
        applied[pname] = entry
    return applied


def recover_awq_scales(model, artifacts_dir: str, metadata: Dict, verify_sha: bool = True) -> Dict:
    """Per-consumer AWQ scale vectors from the norm-gain edits, taken while the model
    is still pristine: s = (1 + w_orig) / (1 + w_edited), or the pinned
    `awq_scale_file` when the entry records one. Scales must be finite, in (0, 1 + 2e-3],
    and agree within 2 % with the consumer metadata's s_min / s_max / s_mean.
    Follows palettized_modules.py:3130-3262."""
    doc = _norm_doc(artifacts_dir)
    edits = (doc or {}).get("edits") or {}
    art = artifacts.ArtifactDir(artifacts_dir, verify_sha)
    named = dict(model.named_parameters())
    tensors = metadata.get("tensors") or {}
    out: Dict = {}
    for pname, entry in edits.items():
        try:
            alpha = float(entry.get("alpha", 0.0) or 0.0)
        except (TypeError, ValueError):
            alpha = 0.0
        if alpha <= 0.0:
            continue
        if pname not in named:
            raise KeyError(f"recover_awq_scales: parameter {pname!r} (norm edit, alpha={alpha}) not "
                           f"found in the loaded model")
        w0 = named[pname].detach().float().cpu()
        if entry.get("awq_scale_file"):
            art.check_sha(entry["awq_scale_file"], entry.get("awq_scale_sha256"), f"awq_recover:{pname}")
            s = torch.from_numpy(np.ascontiguousarray(np.load(art.file(entry["awq_scale_file"])))).float().reshape(-1)
            if s.shape != w0.reshape(-1).shape:
                raise ValueError(f"awq_recover:{pname}: recorded AWQ scale shape {tuple(s.shape)} != "
                                 f"the norm parameter's {tuple(w0.reshape(-1).shape)}")
        else:
            art.check_sha(entry["file"], entry.get("sha256"), f"awq_recover:{pname}")
            gamma = torch.from_numpy(np.ascontiguousarray(np.load(art.file(entry["file"])))).float()
            if gamma.shape != w0.shape:
                raise ValueError(f"awq_recover:{pname}: edited-gain shape {tuple(gamma.shape)} != "
                                 f"the model's {tuple(w0.shape)}")
            gain = 1.0 + gamma
            if bool((gain < 0).any()):
                raise ValueError(f"awq_recover:{pname}: 1 + w_edited has negative entries; not a "
                                 f"zero-centered RMSNorm gain fold")
            s = (1.0 + w0) / gain.clamp(min=1e-6)
        if not torch.isfinite(s).all() or bool((s <= 0).any()) or float(s.max()) > 1.0 + 2e-3:
            raise ValueError(f"awq_recover:{pname}: recovered AWQ scales out of the production range "
                             f"(0, 1] — min {float(s.min()):.4g}, max {float(s.max()):.4g}")
        for consumer in entry.get("consumers") or []:
            awq = (tensors.get(str(consumer)) or {}).get("awq") or {}
            if awq.get("applied"):
                for key, val in (("s_min", float(s.min())), ("s_max", float(s.max())),
                                 ("s_mean", float(s.mean()))):
                    rec = awq.get(key)
                    if rec is not None and abs(val - float(rec)) > 0.02 * max(1.0, abs(float(rec))):
                        raise ValueError(f"awq_recover:{consumer}: recovered {key}={val:.4g} != the "
                                         f"metadata's {float(rec):.4g} (>2%)")
            out.setdefault(str(consumer), s)
    return out


def load_quant_model(artifacts_dir, model_name, device, residual=False, dtype=None, forward="kernel",
                     awq_compensation=True, heads_dir=None, use_m1m2=True, m1m2_mem_size=128,
                     m1m2_gates_path=None, *, verify_sha=True):
    """Returns (model, metadata). Positional order and defaults are those of the reference's
    loader (src/scripts/loader.py:17-21); `verify_sha` is an added keyword.

    model_name: a checkpoint name or path (handed to transformers' AutoModelForCausalLM), or —
    since no checkpoint travels with this package — an nn.Module, or a zero-argument callable
    that builds one.

    use_m1m2 / m1m2_mem_size / m1m2_gates_path: the M1/M2 memories live in the reference's
    vendored model classes, which this package does not carry. With the reference's default
    (use_m1m2=True, no gates file) those memories start from zero-initialised gates and leave
    the model's outputs bit-unchanged, so the default is served by not attaching them. A gates
    file would change the outputs and cannot be honoured: it is refused."""
    if forward not in ("kernel", "reference"):
        raise ValueError(f"forward must be 'kernel' or 'reference', got {forward!r}")
    if m1m2_gates_path:
        raise NotImplementedError(
            "m1m2_gates_path: trained M1/M2 gates need the reference's vendored model classes, "
            "which this package does not carry; load without a gates file")
    model = model_name
    if dtype is None:
        dtype = torch.float16
    metadata = artifacts.load_metadata(artifacts_dir)
    if isinstance(model, str):
        from transformers import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(model, dtype=dtype, low_cpu_mem_usage=True)
    elif not isinstance(model, torch.nn.Module) and callable(model):
        model = model()
    if not isinstance(model, torch.nn.Module):
        raise TypeError("model must be an nn.Module, a callable that builds one, or a checkpoint path")
    model = model.to(dtype)
    awq_scales: Dict = {}
    if awq_compensation:
        awq_scales = recover_awq_scales(model, artifacts_dir, metadata, verify_sha)   # pristine model
    apply_norm_gain_edits(model, artifacts_dir, verify_sha)
    artifacts.replace_linear_with_palettized(model, metadata, artifacts_dir, residual=residual,
                                             reference=(forward == "reference"),
                                             verify_sha=verify_sha, awq_scales=awq_scales,
                                             heads_dir=heads_dir)
    model = model.to(device)
    model.eval()
    return model, metadata
