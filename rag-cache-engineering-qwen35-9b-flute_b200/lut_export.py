"""Palette-set codec: carries the (fine-tuned) palettes of a model's PalettizedLinear modules
through a directory of `.npz` files plus `manifest.json`, interoperable with the reference's
codec (src/rag/lut_export.py: `export_luts`, `import_luts`). Code blobs never change under
fine-tuning; only palettes travel. The kernels read `module.lut` / `module.lut2` on every
forward, so an import takes effect on the next call.

Written from the file format, which is all the two sides share:

  <dir>/<module name, dots doubled to "__", other odd characters to "_">.npz   (no pickle)
      lut            float16 [groups, 2**bitwidth]
      lut2           float16 [groups, 2**bitwidth2]       only with a second stream
      bitwidth, bitwidth2, group_size, N, K              int64 scalars
      rotation_seed, rotation_k (int64), fold_order (str) only when the module has them
      code_sha256    sha256 hex of: lut bytes, lut2 bytes (if any), then the text
                     "bitwidth=4|bitwidth2=4|...|has_stream2=False" (repr of each value, in the
                     key order of GEOMETRY_KEYS)
      header         JSON text {version, exported_utc, module, extra_meta}
  <dir>/manifest.json
      {version, n_modules, files {module: file}, sha256 {file: whole-file digest},
       code_sha256 {module: digest}, exported_utc, extra_meta}
"""
from __future__ import annotations

import hashlib
import json
import os
import re
from dataclasses import dataclass
from datetime import datetime, timezone
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

from .palettized_modules import PalettizedLinear

__all__ = ["LUT_EXPORT_VERSION", "export_luts", "import_luts", "iter_palettized_linears"]

LUT_EXPORT_VERSION = 1
MANIFEST_NAME = "manifest.json"
# the digest text lists the geometry in exactly this order
GEOMETRY_KEYS = ("bitwidth", "bitwidth2", "group_size", "N", "K", "rotation_seed", "rotation_k",
                 "fold_order", "has_stream2")
SCALAR_KEYS = ("bitwidth", "bitwidth2", "group_size", "N", "K")


def iter_palettized_linears(root) -> Iterator[Tuple[str, PalettizedLinear]]:
    """(dotted name, module) for every PalettizedLinear below `root`, including the members of
    merged QKV and fused MLP wrappers."""
    return ((n, m) for n, m in root.named_modules() if isinstance(m, PalettizedLinear))


def _sha256_file(path: str) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            piece = f.read(4 << 20)
            if not piece:
                return digest.hexdigest()
            digest.update(piece)


def _file_name(module_name: str) -> str:
    stem = re.sub(r"[^A-Za-z0-9_.-]+", "_", module_name).replace(".", "__")
    if not stem:
        raise ValueError(f"lut_export: module name {module_name!r} leaves no file name")
    return stem + ".npz"


class _Rejected(ValueError):
    """An entry of an export directory that cannot be installed."""


@dataclass
class PaletteRecord:
    """The palettes of one module with the geometry they belong to."""
    lut: np.ndarray
    lut2: Optional[np.ndarray]
    geometry: Dict

    @staticmethod
    def geometry_of(mod: PalettizedLinear) -> Dict:
        opt = lambda v: None if v is None else int(v)
        return dict(bitwidth=int(mod.bitwidth), bitwidth2=int(mod.bitwidth2), group_size=int(mod.group_size),
                    N=int(mod.N), K=int(mod.K), rotation_seed=opt(mod.rotation_seed),
                    rotation_k=opt(mod.rotation_k), fold_order=mod.fold_order,
                    has_stream2=bool(mod.has_stream2))

    @classmethod
    def of_module(cls, mod: PalettizedLinear) -> "PaletteRecord":
        grab = lambda t: np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float16)
        return cls(grab(mod.lut), None if mod.lut2 is None else grab(mod.lut2), cls.geometry_of(mod))

    def digest(self) -> str:
        h = hashlib.sha256(np.ascontiguousarray(self.lut, dtype=np.float16).tobytes())
        if self.lut2 is not None:
            h.update(np.ascontiguousarray(self.lut2, dtype=np.float16).tobytes())
        h.update("|".join(f"{k}={self.geometry[k]!r}" for k in GEOMETRY_KEYS).encode("utf-8"))
        return h.hexdigest()

    def save(self, path: str, header: Dict) -> None:
        arrays = {k: np.int64(self.geometry[k]) for k in SCALAR_KEYS}
        arrays["lut"] = self.lut
        if self.lut2 is not None:
            arrays["lut2"] = self.lut2
        arrays.update({k: np.int64(self.geometry[k]) for k in ("rotation_seed", "rotation_k")
                       if self.geometry[k] is not None})
        if self.geometry["fold_order"] is not None:
            arrays["fold_order"] = np.array(self.geometry["fold_order"])
        arrays["code_sha256"] = np.array(self.digest())
        arrays["header"] = np.array(json.dumps(header, sort_keys=True))
        np.savez(path, **arrays)

    @classmethod
    def load(cls, path: str, label: str) -> Tuple["PaletteRecord", str, Dict]:
        """(record, recorded digest, header) of one .npz; _Rejected if it is not one of ours."""
        with np.load(path) as z:
            have = set(z.files)
            lacking = sorted(set(SCALAR_KEYS + ("lut", "code_sha256", "header")) - have)
            if lacking:
                raise _Rejected(f"import_luts: {label} lacks the arrays {lacking}; it was not written by export_luts")
            geometry = {k: int(z[k].item()) for k in SCALAR_KEYS}
            for k in ("rotation_seed", "rotation_k"):
                geometry[k] = int(z[k].item()) if k in have else None
            geometry["fold_order"] = str(z["fold_order"].item()) if "fold_order" in have else None
            lut2 = np.asarray(z["lut2"]) if "lut2" in have else None
            geometry["has_stream2"] = lut2 is not None
            try:
                recorded = str(z["code_sha256"].item())
                header = json.loads(str(z["header"].item()))
            except (TypeError, ValueError) as err:
                raise _Rejected(f"import_luts: {label}: digest or header cannot be read ({err})") from err
            return cls(np.asarray(z["lut"]), lut2, geometry), recorded, header

    def problems_for(self, mod: PalettizedLinear, name: str) -> List[str]:
        """Why this record does not fit the live module (empty: it fits)."""
        out = []
        live = self.geometry_of(mod)
        if live != self.geometry:
            differing = {k: (self.geometry[k], live[k]) for k in GEOMETRY_KEYS if self.geometry[k] != live[k]}
            out.append(f"import_luts: {name!r}: geometry of the file and of the model differ (file, model): {differing}")
        for label, mine, theirs in (("lut", self.lut, mod.lut), ("lut2", self.lut2, mod.lut2)):
            if (mine is None) != (theirs is None):
                out.append(f"import_luts: {name!r}: {label} is present on one side only")
            elif mine is not None and (mine.dtype != np.float16 or tuple(mine.shape) != tuple(theirs.shape)):
                out.append(f"import_luts: {name!r}: {label} in the file is {mine.dtype} {tuple(mine.shape)}, "
                           f"the model holds float16-grid {tuple(theirs.shape)}")
        return out

    def install(self, mod: PalettizedLinear) -> None:
        """Replace the module's palettes; dtype and device of the live buffers are kept (a model
        served in bfloat16 gets the float16 grid rounded once, as at load time)."""
        for label, arr in (("lut", self.lut), ("lut2", self.lut2)):
            if arr is None:
                continue
            old = getattr(mod, label)
            fresh = torch.from_numpy(np.ascontiguousarray(arr)).to(dtype=old.dtype, device=old.device)
            mod.register_buffer(label, fresh, persistent=False)


def export_luts(model, out_dir: str, extra_meta: Optional[dict] = None) -> dict:
    """Write every PalettizedLinear's float16 palettes under `model` to `out_dir` (one .npz per
    module + manifest.json) and return the manifest. Only the float16 deployment grid is
    exported: a palette in another dtype is refused."""
    meta = {} if extra_meta is None else extra_meta
    if not isinstance(meta, dict):
        raise TypeError(f"export_luts: extra_meta is a {type(extra_meta).__name__}; a dict (or None) is expected")
    try:
        json.dumps(meta)
    except (TypeError, ValueError) as err:
        raise ValueError(f"export_luts: extra_meta goes into manifest.json and must be JSON-serializable: {err}") from err
    modules = list(iter_palettized_linears(model))
    if not modules:
        raise ValueError("export_luts: the model holds no PalettizedLinear, so there is nothing to write")
    off_grid = [(name, label, str(t.dtype)) for name, mod in modules
                for label, t in (("lut", mod.lut), ("lut2", mod.lut2)) if t is not None and t.dtype != torch.float16]
    if off_grid:
        raise RuntimeError(f"export_luts: palettes must be on the fp16 deployment grid; these are not: {off_grid}")
    names = {}
    for name, _ in modules:
        fname = _file_name(name)
        if fname in names:
            raise ValueError(f"export_luts: modules {names[fname]!r} and {name!r} would both be written to {fname!r}")
        names[fname] = name
    os.makedirs(out_dir, exist_ok=True)
    when = datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")
    manifest = {"version": LUT_EXPORT_VERSION, "n_modules": len(modules), "files": {}, "sha256": {},
                "code_sha256": {}, "exported_utc": when, "extra_meta": meta}
    for name, mod in modules:
        fname = _file_name(name)
        record = PaletteRecord.of_module(mod)
        path = os.path.join(out_dir, fname)
        record.save(path, {"version": LUT_EXPORT_VERSION, "exported_utc": when, "module": name, "extra_meta": meta})
        manifest["files"][name] = fname
        manifest["sha256"][fname] = _sha256_file(path)
        manifest["code_sha256"][name] = record.digest()
    with open(os.path.join(out_dir, MANIFEST_NAME), "w", encoding="utf-8") as f:
        json.dump(manifest, f, indent=2, sort_keys=True)
    return manifest


def _read_manifest(out_dir: str) -> Dict:
    path = os.path.join(out_dir, MANIFEST_NAME)
    if not os.path.isfile(path):
        raise ValueError(f"import_luts: {out_dir} has no {MANIFEST_NAME}; it is not an export directory")
    try:
        with open(path, encoding="utf-8") as f:
            manifest = json.load(f)
    except json.JSONDecodeError as err:
        raise ValueError(f"import_luts: {path} does not parse as JSON ({err})") from err
    if int(manifest.get("version", -1)) != LUT_EXPORT_VERSION:
        raise ValueError(f"import_luts: manifest version is {manifest.get('version')!r}, this codec reads "
                         f"version {LUT_EXPORT_VERSION}")
    if not isinstance(manifest.get("files"), dict) or not manifest["files"]:
        raise ValueError(f"import_luts: {path} lists no files")
    return manifest


def _install_one(mod: Optional[PalettizedLinear], name: str, fname: str, out_dir: str, manifest: Dict) -> None:
    if mod is None:
        raise _Rejected(f"import_luts: the manifest names {name!r}, but the model has no live PalettizedLinear there")
    path = os.path.join(out_dir, fname)
    if not os.path.isfile(path):
        raise _Rejected(f"import_luts: the manifest lists {fname}, which is not in {out_dir}")
    listed = (manifest.get("sha256") or {}).get(fname)
    actual = _sha256_file(path)
    if listed != actual:
        raise _Rejected(f"import_luts: sha256 mismatch on {fname} (manifest {listed}, file {actual})")
    record, recorded, header = PaletteRecord.load(path, fname)
    if int(header.get("version", -1)) != LUT_EXPORT_VERSION:
        raise _Rejected(f"import_luts: {fname} was written as version {header.get('version')!r}, "
                        f"this codec reads version {LUT_EXPORT_VERSION}")
    if recorded != record.digest():
        raise _Rejected(f"import_luts: the palettes in {fname} do not hash to the digest stored beside them")
    problems = record.problems_for(mod, name)
    if problems:
        raise _Rejected("; ".join(problems))
    record.install(mod)


def import_luts(model, out_dir: str, strict: bool = True) -> dict:
    """Install the palette set of `out_dir` into `model`. Every entry is verified first (file
    digest, format version, content digest, geometry and palette shapes against the live module).
    strict: any problem raises, and manifest and model must name the same modules; otherwise
    problems are collected. Returns {"loaded": [...], "checked": n, "mismatches": [...]}."""
    manifest = _read_manifest(str(out_dir))
    live = dict(iter_palettized_linears(model))
    report = {"loaded": [], "checked": len(manifest["files"]), "mismatches": []}

    def complain(message: str, cause=None):
        if strict:
            raise ValueError(message) from cause
        report["mismatches"].append(message)
    for name, fname in manifest["files"].items():
        try:
            _install_one(live.get(name), name, str(fname), str(out_dir), manifest)
        except _Rejected as err:
            complain(str(err), err)
        else:
            report["loaded"].append(name)
    orphans = sorted(set(live) - set(manifest["files"]))
    if orphans:
        complain(f"import_luts: palettized modules of the model that are not covered by the manifest: {orphans}")
    return report
