"""Reader of a palettization artifact directory and the module swap that puts
the B200 LUT kernels behind a model's Linear layers.

On-disk contract (the reference's, src/scripts/palettized_modules.py:229-343,
2411-2724, 2866-3027): `metadata.json` holds `{"tensors": {name: meta}}`. A
tensor meta names an idxN blob `<stem>.idx{b}[.<tag>]` (`index_file`), a float16
palette file (`lut_file`, n_groups x 2^b values), `bitwidth`, `group_size`,
`indices_layout` ("idx1".."idx4"), `dense_shape` [N, K], optional sha256 digests,
an optional second stream (`streams`: [base entry, {file, sha256, sha256_lut,
n_groups, gs, bitwidth}]), an optional low-rank residual (`residual`: resA_file
[N, r], resB_file [r, K], float16) and an optional `rotation` {seed, k}. A fused
QKV tensor carries `components` {"Q","K","V"} of such metas without a
`dense_shape` of their own (N follows from `packed_len_bytes`).

Behaviour kept from the reference: layout name, file name and `bitwidth` must
agree; byte counts are checked; digests are verified; a recorded `group_size`
is honoured when it is consistent with the palette's row count
(n_groups == ceil(N / gs)) and otherwise replaced, with a note, by
ceil(N / n_groups); a declared second stream whose files are missing is an
error, never a silent single-stream load.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn

from .palettized_modules import (FusedPalettizedMLP, PalettizedEmbedding, PalettizedLinear,
                                 SplitQKV)

_IDX_NAME = re.compile(r"^(?P<stem>.*)\.idx(?P<bits>[1-4])(?P<tag>\.[^./]+)?$")
HEAD_TENSORS = ("model.lm_head.weight", "model.embed_tokens.weight")


def load_metadata(artifacts_dir: str) -> Dict:
    with open(os.path.join(artifacts_dir, "metadata.json")) as f:
        return json.load(f)


def parse_index_name(name) -> Optional[Tuple[str, int, str]]:
    """(stem, bits, tag) of an idxN artifact file name, None for anything else."""
    if not isinstance(name, str) or "/" in name:
        return None
    m = _IDX_NAME.match(name)
    if m is None:
        return None
    return m.group("stem"), int(m.group("bits")), m.group("tag") or ""


def lut_name_of(index_file: str) -> Optional[str]:
    """`<stem>.idx{b}` -> `<stem>.lut_scalar`; a stream tag carries over."""
    parsed = parse_index_name(index_file)
    if parsed is None:
        return None
    stem, _, tag = parsed
    return stem + ".lut_scalar" + tag


def layout_bits(layout) -> int:
    if isinstance(layout, str) and re.fullmatch(r"idx[1-4]", layout):
        return int(layout[3])
    raise ValueError(f"not an idxN layout name: {layout!r}")


def validate_indices_layout(meta: Dict, ctx: str) -> int:
    """Layout string, file name and bitwidth field must name the same width."""
    raw = meta.get("indices_layout") or meta.get("layout")
    try:
        bits = layout_bits(raw)
    except ValueError:
        raise ValueError(f"{ctx}: indices_layout={raw!r} is not an idxN layout ('idx1'..'idx4'); "
                         f"older artifact generations are not readable") from None
    parsed = parse_index_name(str(meta.get("index_file", "")))
    if parsed is None:
        raise ValueError(f"{ctx}: index file {meta.get('index_file')!r} is not an idxN artifact")
    if parsed[1] != bits:
        raise ValueError(f"{ctx}: index file {meta['index_file']!r} declares idx{parsed[1]} but "
                         f"indices_layout={raw!r}; the two must agree")
    if meta.get("bitwidth") is not None and int(meta["bitwidth"]) != bits:
        raise ValueError(f"{ctx}: metadata bitwidth {meta['bitwidth']} != the layout's {bits} bits")
    return bits


class ArtifactDir:
    """One artifact directory: file access with digest checks and the per-swap
    record of stale `group_size` fields."""

    def __init__(self, path: str, verify_sha: bool = True):
        self.path, self.verify_sha = path, verify_sha
        self.gs_notes: List[tuple] = []

    def file(self, name: str) -> str:
        return os.path.join(self.path, name)

    def check_sha(self, name: str, expected: Optional[str], ctx: str) -> None:
        if not self.verify_sha or not expected:
            return
        h = hashlib.sha256()
        with open(self.file(name), "rb") as f:
            for block in iter(lambda: f.read(1 << 22), b""):
                h.update(block)
        if h.hexdigest() != expected:
            raise ValueError(f"{ctx}: SHA256 mismatch for {self.file(name)} "
                             f"(metadata {expected[:16]}..., got {h.hexdigest()[:16]}...)")

    # ---------------------------------------------------------------- one stream
    def read_stream(self, meta: Dict, ctx: str, shape=None):
        """(blob uint8, palette [n_groups, 2^b] f16, bits, group_size, N, K)."""
        bits_layout = validate_indices_layout(meta, ctx)
        self.check_sha(meta["index_file"], meta.get("sha256_idx"), ctx)
        self.check_sha(meta["lut_file"], meta.get("sha256_lut"), ctx)
        blob = np.fromfile(self.file(meta["index_file"]), dtype=np.uint8)
        lut = np.fromfile(self.file(meta["lut_file"]), dtype=np.float16)
        bits = int(meta["bitwidth"]) if meta.get("bitwidth") is not None else bits_layout
        entries = 1 << bits
        if lut.size % entries:
            raise ValueError(f"{ctx}: LUT size {lut.size} not divisible by palette size {entries}")
        n_groups = lut.size // entries
        N, K = shape if shape is not None else meta.get("dense_shape", [None, None])
        if N is None:
            raise ValueError(f"{ctx}: metadata missing dense_shape")
        N, K = int(N), int(K)
        meta_gs = int(meta["group_size"])
        group_size = meta_gs
        if n_groups > 0:
            derived = -(-N // n_groups)
            if not (meta_gs > 0 and n_groups == -(-N // meta_gs)):
                group_size = derived
                if meta_gs > 0 and meta_gs != derived:
                    self.note_gs(ctx, meta_gs, n_groups, N, derived)
        expected = N * ((K * bits + 7) // 8)
        if blob.size != expected:
            raise ValueError(f"{ctx}: index file {meta['index_file']} has {blob.size} B, expected "
                             f"N*K_packed = {expected} B (N={N}, K={K}, bitwidth={bits})")
        return (torch.from_numpy(blob), torch.from_numpy(lut).view(n_groups, entries), bits,
                group_size, N, K)

    def note_gs(self, ctx, meta_gs, n_groups, N, derived) -> None:
        self.gs_notes.append((ctx, meta_gs, n_groups, N, derived))
        if len(self.gs_notes) == 1:
            print(f"[artifacts] {ctx}: metadata group_size {meta_gs} is inconsistent with the LUT "
                  f"geometry (n_groups={n_groups}, N={N} -> derived {derived}); using the derived "
                  f"value", flush=True)

    def summarize_gs(self) -> None:
        if len(self.gs_notes) > 1:
            first = self.gs_notes[0]
            print(f"  [GS] group_size metadata mismatch on {len(self.gs_notes)} tensor component(s) "
                  f"(first: {first[0]}: gs {first[1]} vs derived {first[4]}); the LUT geometry is "
                  f"trusted for every one of them", flush=True)
        self.gs_notes = []

    # ------------------------------------------------------------- second stream
    def read_stream2(self, meta: Dict, ctx: str, N: int, K: int, bits: int, group_size: int):
        streams = meta.get("streams")
        if not isinstance(streams, list) or len(streams) < 2:
            raise ValueError(f"{ctx}: metadata 'streams' must be a list with at least 2 entries, "
                             f"got {streams!r}; refusing an ambiguous stream set")
        base = streams[0] if isinstance(streams[0], dict) else {}
        if base.get("file") != meta.get("index_file"):
            raise ValueError(f"{ctx}: streams[0] file {base.get('file')!r} != the meta's index_file "
                             f"{meta.get('index_file')!r}; the first entry must describe the base "
                             f"stream")
        entry = streams[1]
        if not isinstance(entry, dict) or "file" not in entry:
            raise ValueError(f"{ctx}: stream-2 entry must be a dict carrying 'file' (got {entry!r})")
        name2 = str(entry["file"])
        parsed = parse_index_name(name2)
        if parsed is None:
            raise ValueError(f"{ctx}: stream-2 file {name2!r} is not a (tagged) idxN artifact name")
        bits2 = parsed[1]
        if entry.get("bitwidth") is not None and int(entry["bitwidth"]) != bits2:
            raise ValueError(f"{ctx}: stream-2 entry bitwidth {entry['bitwidth']} != the file name's "
                             f"idx{bits2} ({name2!r})")
        lut2_name = lut_name_of(name2)
        for fname in (name2, lut2_name):
            if not os.path.exists(self.file(fname)):
                raise ValueError(f"{ctx}: metadata declares {len(streams)} streams but stream-2 member "
                                 f"{fname!r} is missing (expected {self.file(fname)}); the two-stream "
                                 f"artifact set is incomplete (never a silent single-stream fallback)")
        member = {"index_file": name2, "lut_file": lut2_name, "sha256_idx": entry.get("sha256"),
                  "sha256_lut": entry.get("sha256_lut"), "bitwidth": bits2,
                  "group_size": int(entry.get("gs", group_size)), "indices_layout": f"idx{bits2}"}
        blob2, lut2, _, _, _, _ = self.read_stream(member, f"{ctx}:stream2", shape=(N, K))
        if entry.get("n_groups") is not None and int(entry["n_groups"]) != lut2.shape[0]:
            raise ValueError(f"{ctx}: stream-2 n_groups {entry['n_groups']} != the LUT's "
                             f"{lut2.shape[0]} rows (corrupt stream-2 metadata)")
        return blob2, lut2, bits2

    # ------------------------------------------------------------------ residual
    def read_residual(self, meta: Dict, ctx: str, N: int, K: int):
        res = meta.get("residual")
        if not res:
            return None, None
        self.check_sha(res["resA_file"], res.get("sha256_resA"), ctx)
        self.check_sha(res["resB_file"], res.get("sha256_resB"), ctx)
        rank = int(res["rank"])
        A = torch.from_numpy(np.fromfile(self.file(res["resA_file"]), dtype=np.float16)).view(N, rank)
        B = torch.from_numpy(np.fromfile(self.file(res["resB_file"]), dtype=np.float16)).view(rank, K)
        return A, B

    # ------------------------------------------------------------------- modules
    def _linear(self, meta: Dict, ctx: str, shape, bias, residual: bool, reference: bool,
                awq_scale, fold_order) -> PalettizedLinear:
        blob, lut, bits, gs, N, K = self.read_stream(meta, ctx, shape=shape)
        blob2 = lut2 = bits2 = None
        if meta.get("streams"):
            blob2, lut2, bits2 = self.read_stream2(meta, ctx, N, K, bits, gs)
        resA = resB = None
        if residual:
            resA, resB = self.read_residual(meta, ctx, N, K)
        rot = meta.get("rotation")
        return PalettizedLinear(blob, lut, bits, gs, N, K, bias=bias, resA=resA, resB=resB,
                                indices2=blob2, lut2=lut2, bitwidth2=bits2, reference=reference,
                                rotation_seed=rot["seed"] if rot else None,
                                rotation_k=rot["k"] if rot else None,
                                awq_scale=awq_scale, fold_order=fold_order)

    def load_embedding(self, meta: Dict, residual: bool = True) -> PalettizedEmbedding:
        """PalettizedEmbedding of an embed_tokens entry: both declared streams, the residual
        pair when present, the rotation record of a tied head set (reference
        load_palettized_embedding, palettized_modules.py:2731-2768)."""
        ctx = meta.get("var", "?")
        if "components" in meta:
            raise ValueError(f"{ctx}: an embedding meta carries no QKV components (embed_tokens is "
                             f"a single matrix, never a fused projection); refusing to guess a "
                             f"component split")
        blob, lut, bits, gs, N, K = self.read_stream(meta, ctx)
        resA = resB = None
        if residual:
            resA, resB = self.read_residual(meta, ctx, N, K)
        blob2 = lut2 = bits2 = None
        if meta.get("streams"):
            blob2, lut2, bits2 = self.read_stream2(meta, ctx, N, K, bits, gs)
        rot = meta.get("rotation")
        return PalettizedEmbedding(blob, lut, bits, gs, N, K, indices2=blob2, lut2=lut2,
                                   bitwidth2=bits2, resA=resA, resB=resB,
                                   rotation_seed=rot["seed"] if rot else None,
                                   rotation_k=rot["k"] if rot else None)

    def load_tied_pair(self, lm_meta: Dict, embed_meta: Optional[Dict], residual: bool = True,
                       reference: bool = False, awq_scales: Optional[Dict] = None):
        """(PalettizedLinear, PalettizedEmbedding) over ONE artifact set: read once through
        the lm_head's metadata, the embedding built on the same tensors; both metas must
        describe the same member set (reference load_tied_pair, :2792-2872)."""
        lm_var = str(lm_meta.get("var", "?"))
        if embed_meta is None:
            embed_meta, emb_var = lm_meta, f"{lm_var}(tied)"
        else:
            emb_var = str(embed_meta.get("var", "?"))
        if lm_meta.get("tied") is not True:
            raise ValueError(f"load_tied_pair({lm_var}, {emb_var}): the lm_head metadata does not "
                             f"carry the writer's \"tied\": true record — this is not a "
                             f"one-artifact-set tied entry; load each consumer separately")
        if "components" in lm_meta:
            raise ValueError(f"load_tied_pair({lm_var}, {emb_var}): a tied head is a single matrix, "
                             f"never a QKV component split")
        rows_l, rows_e = tied_member_rows(lm_meta), tied_member_rows(embed_meta)
        if rows_l != rows_e:
            detail = "the member sets differ"
            for i in range(max(len(rows_l), len(rows_e))):
                a = rows_l[i] if i < len(rows_l) else None
                b = rows_e[i] if i < len(rows_e) else None
                if a != b:
                    detail = (f"member {a[0] if a else b[0]}: lm_head expects {a[1:] if a else None}, "
                              f"embed expects {b[1:] if b else None}")
                    break
            raise ValueError(f"load_tied_pair({lm_var}, {emb_var}): the two consumers' metadata "
                             f"describe different artifact sets — {detail}; refusing to serve one "
                             f"artifact set to disagreeing consumers")
        lm = self.load_weight(lm_meta, residual=residual, reference=reference, awq_scales=awq_scales)
        return lm, PalettizedEmbedding.tied_to(lm)

    def load_weight(self, meta: Dict, bias=None, residual: bool = False, reference: bool = False,
                    awq_scales: Optional[Dict] = None):
        """PalettizedLinear, or SplitQKV for a fused QKV tensor (the original bias is
        sliced per component)."""
        name = meta.get("var", "?")
        scale, fold = _awq_for(meta, awq_scales)
        if "components" not in meta:
            return self._linear(meta, name, None, None if bias is None else bias.clone(),
                                residual, reference, scale, fold)
        K = int(meta["dense_shape"][1])
        fold = fold or (meta.get("awq") or {}).get("fold_order")
        parts = []
        for key in ("Q", "K", "V"):
            cm = meta["components"][key]
            n = int(cm["packed_len_bytes"]) * 8 // (K * int(cm["bitwidth"]))
            parts.append(self._linear(cm, f"{name}:{key}", (n, K), None, residual, reference,
                                      scale, fold))
        if bias is not None:
            off = 0
            for m in parts:
                m.bias = nn.Parameter(bias[off:off + m.N].clone())
                off += m.N
            if off != bias.shape[0]:
                raise ValueError(f"{name}: bias length {bias.shape[0]} != sum of component N ({off})")
        return SplitQKV(*parts)


def tied_member_rows(meta: Dict):
    """(member, file, expected sha256) rows of every artifact member a consumer's metadata
    describes; two consumers of one tied set must produce equal rows (reference
    _tied_member_rows, palettized_modules.py:2771-2789)."""
    rows = [("index_file", meta.get("index_file"), meta.get("sha256_idx")),
            ("lut_file", meta.get("lut_file"), meta.get("sha256_lut"))]
    for i, entry in enumerate(meta.get("streams") or []):
        rows.append((f"streams[{i}].idxN", entry.get("file"), entry.get("sha256")))
        rows.append((f"streams[{i}].lut_scalar", entry.get("file"), entry.get("sha256_lut")))
    res = meta.get("residual")
    if res:
        rows.append(("resA_file", res.get("resA_file"), res.get("sha256_resA")))
        rows.append(("resB_file", res.get("resB_file"), res.get("sha256_resB")))
    return rows


def _awq_for(meta: Dict, awq_scales: Optional[Dict]):
    """(K-vector scale, fold order) recorded for a tensor, (None, None) when unscaled."""
    if not awq_scales:
        return None, None
    s = awq_scales.get(meta.get("var") or meta.get("name"))
    if s is None:
        return None, None
    order = (meta.get("awq") or {}).get("fold_order") or (meta.get("rotation") or {}).get("order")
    return s, order


def load_palettized_weight(tensor_meta: Dict, artifacts_dir: str, bias=None, residual: bool = False,
                           reference: bool = False, verify_sha: bool = True,
                           awq_scales: Optional[Dict] = None):
    """The reference's per-tensor entry (palettized_modules.py:2619-2724)."""
    return ArtifactDir(artifacts_dir, verify_sha).load_weight(tensor_meta, bias, residual, reference,
                                                             awq_scales)


def load_palettized_embedding(tensor_meta: Dict, artifacts_dir: str, residual: bool = True,
                              verify_sha: bool = True) -> PalettizedEmbedding:
    """The reference's embedding entry (palettized_modules.py:2731-2768)."""
    return ArtifactDir(artifacts_dir, verify_sha).load_embedding(tensor_meta, residual)


def load_tied_pair(lm_head_meta: Dict, embed_meta: Optional[Dict], artifacts_dir: str,
                   residual: bool = True, reference: bool = False, verify_sha: bool = True,
                   awq_scales: Optional[Dict] = None):
    """The reference's tied-pair entry (palettized_modules.py:2792-2872)."""
    return ArtifactDir(artifacts_dir, verify_sha).load_tied_pair(lm_head_meta, embed_meta, residual,
                                                                reference, awq_scales)


# ------------------------------------------------------------------------- swap
def get_layers(model):
    inner = getattr(model, "model", None)
    if inner is not None and hasattr(inner, "layers"):
        return inner.layers
    if inner is not None and hasattr(inner, "language_model"):
        return inner.language_model.layers
    raise AttributeError("Cannot find decoder layers in model structure")


def resolve_module(model, tensor_name: str):
    """(holder module, attribute name) of the Linear that a metadata tensor name
    denotes: `model.layers.<i>.<path>.weight`, or the head names
    `model.lm_head.weight` / `model.embed_tokens.weight` (looked up on the wrapper
    and on its text model; two different modules under one name are refused)."""
    parts = tensor_name.split(".")
    if tensor_name in HEAD_TENSORS:
        leaf = parts[1]
        found = [(label, base) for label, base in (("model", model),
                                                   ("model.model", getattr(model, "model", model)))
                 if hasattr(base, leaf)]
        if not found:
            raise ValueError(f"resolve_module({tensor_name}): no head module named {leaf!r} on the "
                             f"model or its text model")
        first = getattr(found[0][1], leaf)
        for label, base in found[1:]:
            if getattr(base, leaf) is not first:
                raise ValueError(f"resolve_module({tensor_name}): ambiguous — {found[0][0]}.{leaf} "
                                 f"and {label}.{leaf} are different modules; refusing to guess")
        return found[0][1], leaf
    holder = get_layers(model)[int(parts[2])]
    path = parts[3:-1]
    for attr in path[:-1]:
        holder = getattr(holder, attr)
    return holder, path[-1]


def install_fused_mlp(model) -> int:
    """Wrap every MLP block whose gate/up projections are palettized (class name
    `Qwen3_5MLP`, or any module with gate_proj/up_proj/down_proj/act_fn) so that
    decode runs gate + up + SiLU*mul as one launch. FLUTE_NO_MERGE=1 skips it."""
    if os.environ.get("FLUTE_NO_MERGE", "").strip() in ("1", "true", "True"):
        return 0
    todo = []
    for _, parent in model.named_modules():
        for child_name, child in parent.named_children():
            if isinstance(child, FusedPalettizedMLP):
                continue
            gate, up = getattr(child, "gate_proj", None), getattr(child, "up_proj", None)
            down, act = getattr(child, "down_proj", None), getattr(child, "act_fn", None)
            if isinstance(gate, PalettizedLinear) and isinstance(up, PalettizedLinear) \
                    and down is not None and act is not None:
                todo.append((parent, child_name, FusedPalettizedMLP(gate, up, down, act)))
    for parent, child_name, fused in todo:
        setattr(parent, child_name, fused)
    return len(todo)


def replace_linear_with_palettized(model, metadata, artifacts_dir: str, residual: bool = False,
                                   reference: bool = False, verify_sha: bool = True,
                                   awq_scales: Optional[Dict] = None,
                                   heads_dir: Optional[str] = None):
    """Swap every tensor of the metadata for its palettized module, then install
    the fused MLP wrappers (the reference's swap, palettized_modules.py:2921-3027).
    `model.lm_head.weight` is a linear layer like any other (248 320 rows on the 9B model);
    `model.embed_tokens.weight` becomes a PalettizedEmbedding; an lm_head entry that carries
    "tied": true serves both consumers from one artifact set (one copy of the codes on the
    device)."""
    tensors = dict(metadata["tensors"])
    if heads_dir is not None:
        heads = load_metadata(heads_dir)["tensors"]
        for key in HEAD_TENSORS:
            tensors.pop(key, None)
            if key in heads:
                tensors[key] = heads[key]
    art = ArtifactDir(artifacts_dir, verify_sha)
    head_art = None
    for name, meta in tensors.items():
        head_dir = heads_dir if (heads_dir is not None and name in HEAD_TENSORS) else None
        if head_dir is not None and (head_art is None):
            head_art = ArtifactDir(head_dir, verify_sha)
        src = head_art if head_dir is not None else art
        if name == "model.lm_head.weight" and meta.get("tied") is True:
            lm, emb = src.load_tied_pair(meta, None, residual=residual, reference=reference,
                                         awq_scales=awq_scales)
            holder, leaf = resolve_module(model, name)
            setattr(holder, leaf, lm)
            holder, leaf = resolve_module(model, "model.embed_tokens.weight")
            setattr(holder, leaf, emb)
            continue
        holder, leaf = resolve_module(model, name)
        old = getattr(holder, leaf)
        if name == "model.embed_tokens.weight":
            new = src.load_embedding(meta, residual=residual)
        else:
            bias = getattr(old, "bias", None)
            new = src.load_weight(meta, bias=None if bias is None else bias.data, residual=residual,
                                  reference=reference, awq_scales=awq_scales)
        setattr(holder, leaf, new)
        del old
    art.summarize_gs()
    install_fused_mlp(model)
    return model
