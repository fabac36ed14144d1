"""Codec of fine-tuned palette sets: one `.npz` per PalettizedLinear plus a
`manifest.json` (the reference's src/rag/lut_export.py:1-428 — `export_luts`,
`import_luts`). The idxN code blobs never change under fine-tuning, only the palettes do;
this is the channel that carries a new palette set into a loaded model, so that the
kernels serve it on the next forward (they read `module.lut` / `module.lut2` directly).

File contract kept from the reference, so that directories written by either side load on
the other:
  per module `<sanitized name>.npz` (numpy arrays only, no pickle):
    lut (G, 2^bitwidth) float16; lut2 (G, 2^bitwidth2) float16 when a second stream
    exists; bitwidth, bitwidth2, group_size, N, K as int64 scalars; rotation_seed,
    rotation_k, fold_order only when set; code_sha256 = sha256(lut bytes [+ lut2 bytes] +
    canonical config line); header = JSON {version, exported_utc, module, extra_meta}
  manifest.json: {version, n_modules, files {module: file}, sha256 {file: digest},
    code_sha256 {module: digest}, exported_utc, extra_meta}
Import validates, per entry: the whole-file digest, the header version, the content
digest, the geometry against the live module, palette shapes and dtype; `strict=True`
also requires manifest and model to cover each other exactly.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
from datetime import datetime, timezone
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch
from torch import nn

from .palettized_modules import PalettizedLinear

__all__ = ["LUT_EXPORT_VERSION", "export_luts", "import_luts", "iter_palettized_linears"]

LUT_EXPORT_VERSION = 1                      # lut_export.py:72
MANIFEST_NAME = "manifest.json"
# order of the digest's config line (lut_export.py:77-78); never reorder
_CONFIG_KEYS = ("bitwidth", "bitwidth2", "group_size", "N", "K", "rotation_seed", "rotation_k",
                "fold_order", "has_stream2")
_INT_KEYS = ("bitwidth", "bitwidth2", "group_size", "N", "K")
_NPZ_REQUIRED = _INT_KEYS + ("lut", "code_sha256", "header")


class _EntryError(ValueError):
    """One manifest entry failed validation."""


def iter_palettized_linears(root) -> Iterator[Tuple[str, PalettizedLinear]]:
    """(dotted name, module) of every PalettizedLinear under root, the children of merged
    QKV and fused MLP wrappers included (reference palettized_modules.py:3079-3083)."""
    for name, mod in root.named_modules():
        if isinstance(mod, PalettizedLinear):
            yield name, mod


def _module_config(mod) -> Dict:
    return {"bitwidth": int(mod.bitwidth), "bitwidth2": int(mod.bitwidth2),
            "group_size": int(mod.group_size), "N": int(mod.N), "K": int(mod.K),
            "rotation_seed": None if mod.rotation_seed is None else int(mod.rotation_seed),
            "rotation_k": None if mod.rotation_k is None else int(mod.rotation_k),
            "fold_order": mod.fold_order, "has_stream2": bool(mod.has_stream2)}


def _code_digest(lut: np.ndarray, lut2: Optional[np.ndarray], cfg: Dict) -> str:
    """sha256 over the palette bytes and the config line `k=repr(v)|...` (lut_export.py:104-122)."""
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(lut, dtype=np.float16).tobytes())
    if lut2 is not None:
        h.update(np.ascontiguousarray(lut2, dtype=np.float16).tobytes())
    h.update("|".join(f"{k}={cfg[k]!r}" for k in _CONFIG_KEYS).encode("utf-8"))
    return h.hexdigest()


def _file_digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 22), b""):
            h.update(block)
    return h.hexdigest()


def _sanitize(name: str) -> str:
    s = re.sub(r"[^A-Za-z0-9_.-]+", "_", name).replace(".", "__")
    if not s:
        raise ValueError(f"lut_export: cannot sanitize empty module name {name!r}")
    return s


def export_luts(model, out_dir: str, extra_meta: Optional[dict] = None) -> dict:
    """Write the float16 palettes of every PalettizedLinear under `model` to
    `<out_dir>/*.npz` + `<out_dir>/manifest.json`; returns the manifest. Palettes that are
    not float16 are refused (the served grid is the float16 one, lut_export.py:182-190)."""
    if extra_meta is not None and not isinstance(extra_meta, dict):
        raise TypeError(f"export_luts: extra_meta must be a dict or None, got "
                        f"{type(extra_meta).__name__}")
    try:
        json.dumps(extra_meta if extra_meta is not None else {})
    except (TypeError, ValueError) as e:
        raise ValueError(f"export_luts: extra_meta must be JSON-serializable (it lands in "
                         f"manifest.json): {e}") from e
    mods = list(iter_palettized_linears(model))
    if not mods:
        raise ValueError("export_luts: no PalettizedLinear modules under this model — nothing to "
                         "export")
    bad = [(n, str(m.lut.dtype)) for n, m in mods if m.lut.dtype != torch.float16]
    bad += [(n, str(m.lut2.dtype)) for n, m in mods
            if m.lut2 is not None and m.lut2.dtype != torch.float16]
    if bad:
        raise RuntimeError(f"export_luts: LUT buffers must be the fp16 deployment grid: {bad}")
    os.makedirs(out_dir, exist_ok=True)
    stamp = datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")
    files: Dict[str, str] = {}
    sha: Dict[str, str] = {}
    code: Dict[str, str] = {}
    claimed: Dict[str, str] = {}
    for name, mod in mods:
        fname = _sanitize(name) + ".npz"
        if fname in claimed:
            raise ValueError(f"export_luts: sanitized filename collision: {fname!r} for module "
                             f"{name!r} and {claimed[fname]!r} — refusing an ambiguous artifact set")
        claimed[fname] = name
        cfg = _module_config(mod)
        lut = np.ascontiguousarray(mod.lut.detach().cpu().numpy(), dtype=np.float16)
        lut2 = None if mod.lut2 is None else \
            np.ascontiguousarray(mod.lut2.detach().cpu().numpy(), dtype=np.float16)
        digest = _code_digest(lut, lut2, cfg)
        payload = {k: np.int64(cfg[k]) for k in _INT_KEYS}
        payload["lut"] = lut
        if lut2 is not None:
            payload["lut2"] = lut2
        for key in ("rotation_seed", "rotation_k"):
            if cfg[key] is not None:
                payload[key] = np.int64(cfg[key])
        if cfg["fold_order"] is not None:
            payload["fold_order"] = np.array(cfg["fold_order"])
        payload["code_sha256"] = np.array(digest)
        payload["header"] = np.array(json.dumps(
            {"version": LUT_EXPORT_VERSION, "exported_utc": stamp, "module": name,
             "extra_meta": extra_meta or {}}, sort_keys=True))
        path = os.path.join(out_dir, fname)
        np.savez(path, **payload)
        files[name], sha[fname], code[name] = fname, _file_digest(path), digest
    manifest = {"version": LUT_EXPORT_VERSION, "n_modules": len(mods), "files": files, "sha256": sha,
                "code_sha256": code, "exported_utc": stamp, "extra_meta": extra_meta or {}}
    with open(os.path.join(out_dir, MANIFEST_NAME), "w", encoding="utf-8") as f:
        json.dump(manifest, f, indent=2, sort_keys=True)
    return manifest


def _load_entry(path: str, fname: str):
    with np.load(path) as z:
        missing = [k for k in _NPZ_REQUIRED if k not in z.files]
        if missing:
            raise _EntryError(f"import_luts: {fname}: npz is missing keys {missing} — not a "
                              f"lut_export artifact")
        lut = np.asarray(z["lut"])
        lut2 = np.asarray(z["lut2"]) if "lut2" in z.files else None
        cfg = {k: int(z[k].item()) for k in _INT_KEYS}
        cfg["rotation_seed"] = int(z["rotation_seed"].item()) if "rotation_seed" in z.files else None
        cfg["rotation_k"] = int(z["rotation_k"].item()) if "rotation_k" in z.files else None
        cfg["fold_order"] = str(z["fold_order"].item()) if "fold_order" in z.files else None
        cfg["has_stream2"] = lut2 is not None
        try:
            code_sha = str(z["code_sha256"].item())
            header = json.loads(str(z["header"].item()))
        except (ValueError, TypeError) as e:
            raise _EntryError(f"import_luts: {fname}: unreadable code_sha256/header ({e}) — corrupt "
                              f"artifact?") from e
    return lut, lut2, cfg, code_sha, header


def _import_entry(live: Dict[str, PalettizedLinear], name: str, fname: str, out_dir: str,
                  manifest: Dict) -> None:
    mod = live.get(name)
    if mod is None:
        raise _EntryError(f"import_luts: manifest entry {name!r} has no live PalettizedLinear — "
                          f"the artifact set and this model have drifted (strict import requires "
                          f"exact coverage)")
    path = os.path.join(out_dir, fname)
    if not os.path.isfile(path):
        raise _EntryError(f"import_luts: {path} is missing (the manifest lists it)")
    want, got = (manifest.get("sha256") or {}).get(fname), _file_digest(path)
    if want is None or got != want:
        raise _EntryError(f"import_luts: sha256 mismatch for {fname}: manifest {want}, got {got} — "
                          f"the file changed after export")
    lut, lut2, cfg, code_sha, header = _load_entry(path, fname)
    if int(header.get("version", -1)) != LUT_EXPORT_VERSION:
        raise _EntryError(f"import_luts: {fname}: npz header version {header.get('version')!r} != "
                          f"LUT_EXPORT_VERSION {LUT_EXPORT_VERSION} — regenerate the export")
    if code_sha != _code_digest(lut, lut2, cfg):
        raise _EntryError(f"import_luts: {fname}: code sha256 mismatch — the LUT content does not "
                          f"match its recorded digest (corrupt artifact?)")
    live_cfg = _module_config(mod)
    if cfg != live_cfg:
        raise _EntryError(f"import_luts: {name!r}: exported geometry {cfg} != live module geometry "
                          f"{live_cfg} — the artifact set and the model disagree")
    if lut.dtype != np.float16 or tuple(lut.shape) != tuple(mod.lut.shape):
        raise _EntryError(f"import_luts: {name!r}: exported lut shape/dtype {tuple(lut.shape)}/"
                          f"{lut.dtype} != live buffer {tuple(mod.lut.shape)}/float16")
    if lut2 is not None:
        live2 = mod.lut2
        if live2 is None or tuple(lut2.shape) != tuple(live2.shape) or lut2.dtype != np.float16:
            raise _EntryError(f"import_luts: {name!r}: exported lut2 shape/dtype {tuple(lut2.shape)}/"
                              f"{lut2.dtype} does not match the live module")
    elif mod.lut2 is not None:
        raise _EntryError(f"import_luts: {name!r}: the live module has a stream-2 LUT but the "
                          f"artifact has none (lut2)")
    # the live palette's dtype and device are kept (a model served in bfloat16 receives the
    # float16 grid rounded once, exactly as at load time)
    mod.register_buffer("lut", torch.from_numpy(np.ascontiguousarray(lut)).to(
        dtype=mod.lut.dtype, device=mod.lut.device), persistent=False)
    if lut2 is not None:
        mod.register_buffer("lut2", torch.from_numpy(np.ascontiguousarray(lut2)).to(
            dtype=mod.lut2.dtype, device=mod.lut2.device), persistent=False)


def import_luts(model, out_dir: str, strict: bool = True) -> dict:
    """Install an exported palette set into `model` (buffers replaced after digest, geometry
    and shape checks). strict: manifest and live modules must cover each other exactly.
    Returns {"loaded": [names], "checked": n, "mismatches": [messages]}."""
    mpath = os.path.join(out_dir, MANIFEST_NAME)
    if not os.path.isfile(mpath):
        raise ValueError(f"import_luts: no {MANIFEST_NAME} at {mpath} — not an export directory")
    try:
        with open(mpath, encoding="utf-8") as f:
            manifest = json.load(f)
    except json.JSONDecodeError as e:
        raise ValueError(f"import_luts: {mpath} is not valid JSON ({e}) — corrupt manifest") from e
    if int(manifest.get("version", -1)) != LUT_EXPORT_VERSION:
        raise ValueError(f"import_luts: manifest version {manifest.get('version')!r} != "
                         f"LUT_EXPORT_VERSION {LUT_EXPORT_VERSION} — regenerate the export")
    files = manifest.get("files")
    if not isinstance(files, dict) or not files:
        raise ValueError(f"import_luts: {mpath}: manifest has no 'files' mapping — corrupt manifest")
    live = dict(iter_palettized_linears(model))
    loaded: List[str] = []
    mismatches: List[str] = []
    for name, fname in files.items():
        try:
            _import_entry(live, name, str(fname), str(out_dir), manifest)
            loaded.append(name)
        except _EntryError as e:
            if strict:
                raise ValueError(str(e)) from e
            mismatches.append(str(e))
    extra = sorted(n for n in live if n not in files)
    if extra:
        msg = (f"import_luts: live palettized modules not covered by the manifest: {extra} — the "
               f"artifact set and this model have drifted (strict import requires exact coverage)")
        if strict:
            raise ValueError(msg)
        mismatches.append(msg)
    return {"loaded": loaded, "checked": len(files), "mismatches": mismatches}
