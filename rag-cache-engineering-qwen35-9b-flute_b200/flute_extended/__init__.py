"""`flute_extended`-compatible surface over the B200 library.

A caller written against the reference's extension package
(src/flute_extended/flute_extended/__init__.py:138-1109) imports this module in its place:
the same function names, argument order and meaning, the same `*_available()` /
`*_supported()` gates, `gemv_split_hint` and the pair / group-size tables. Everything runs on
libb200lut.so; nothing here computes on the CPU or through torch, except the dense baseline
`qgemm_dense`, which is a plain `torch.matmul` as the reference's benchmark uses.

Differences a caller can observe:
  * fp16 AND bf16 are served (the reference kernels are fp16 only); the activation dtype must
    equal the LUT dtype.
  * The `indices` operands are idxN blobs, as in the reference. This library streams its own
    slab layout, so every distinct blob is converted once, on its device, on first use and the
    converted copy is cached (keyed by the blob's address, size and width; `forget()` drops the
    cache, e.g. after a blob was rewritten in place).
  * The gates describe what THIS library serves, which is a superset of the reference's tables:
    every (b1, b2) width pair, any group size that is 32, 64 or a multiple of 128, any M for
    `qgemm_per_group_lut`, M <= 16 for the decode entries.
  * `rot_signs` / `awq_scale` are honoured by one transform launch in front of the projection
    (the reference fuses the transform into its M = 1 kernels).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _lib
from .. import idxN                                                     # noqa: F401  (flute_extended.idxN)
from ..idxN import pack_idxn, unpack_idxn                               # noqa: F401
from ..palettized_modules import PalettizedLinear, _flags

__all__ = [
    "qgemm_per_group_lut", "qgemm_dense", "qgemm_dual_stream", "qgemm_gemv_stream",
    "qgemm_gemv_splitk_stream", "qgemm_gemv_multi", "qgemm_gemv_mlp",
    "dual_stream_available", "dual_stream_supported", "gemv_stream_available", "gemv_stream_supported",
    "gemv_fht_stream_available", "gemv_fht_stream_supported", "gemv_splitk_available",
    "gemv_splitk_fht_available", "gemv_splitk_supported", "gemv_splitk_fht_supported",
    "gemv_multi_available", "gemv_multi_supported", "gemv_mlp_available", "gemv_mlp_supported",
    "gemv_split_hint", "forget", "pack_idxn", "unpack_idxn", "idxN",
    "DUAL_STREAM_PAIRS", "DUAL_STREAM_GROUP_SIZES", "DUAL_STREAM_MAX_M", "GEMV_STREAM_PAIRS",
    "GEMV_STREAM_GROUP_SIZES", "GEMV_SPLITK_PAIRS", "GEMV_SPLITK_GROUP_SIZES",
    "GEMV_SPLITK_MAX_RESIDUAL_RANK",
]

# ---- tables (names of src/flute_extended/flute_extended/__init__.py:231-242, 345-354, 603-618) ----
_ALL_PAIRS = frozenset((b1, b2) for b1 in range(1, 5) for b2 in range(0, 5))
DUAL_STREAM_PAIRS = _ALL_PAIRS
GEMV_STREAM_PAIRS = _ALL_PAIRS
GEMV_SPLITK_PAIRS = _ALL_PAIRS
_GROUP_SIZES = frozenset({32, 64} | {128 * i for i in range(1, 17)})
DUAL_STREAM_GROUP_SIZES = _GROUP_SIZES
GEMV_STREAM_GROUP_SIZES = _GROUP_SIZES
GEMV_SPLITK_GROUP_SIZES = _GROUP_SIZES
DUAL_STREAM_MAX_M = 16
GEMV_SPLITK_MAX_RESIDUAL_RANK = 4096
_LAYOUT_BITS = {"idx1": 1, "idx2": 2, "idx3": 3, "idx4": 4}


# ---- gates -------------------------------------------------------------------------------------
def _built() -> bool:
    return os.path.exists(_lib.LIB_PATH)


def _shape_ok(bitwidth, bitwidth2, group_size, N, K) -> bool:
    b1, b2 = int(bitwidth), int(bitwidth2) if bitwidth2 else 0
    gs = int(group_size)
    return ((b1, b2) in _ALL_PAIRS and (gs in (32, 64) or (gs >= 128 and gs % 128 == 0))
            and int(N) > 0 and int(N) % 128 == 0 and int(K) > 0 and int(K) % 64 == 0)


def dual_stream_available() -> bool:
    return _built()


def dual_stream_supported(bitwidth, bitwidth2, group_size, N, K) -> bool:
    return _built() and _shape_ok(bitwidth, bitwidth2, group_size, N, K)


def gemv_stream_available() -> bool:
    return _built()


def gemv_stream_supported(bitwidth, bitwidth2, group_size, N, K, M) -> bool:
    return _built() and 1 <= int(M) <= DUAL_STREAM_MAX_M and _shape_ok(bitwidth, bitwidth2, group_size, N, K)


def gemv_fht_stream_available() -> bool:
    return _built()


def gemv_fht_stream_supported(bitwidth, bitwidth2, group_size, N, K, M) -> bool:
    # the transform serves power-of-two segments up to 8192 points
    return gemv_stream_supported(bitwidth, bitwidth2, group_size, N, K, M) and int(K) <= 65536


def gemv_splitk_available() -> bool:
    return _built()


def gemv_splitk_fht_available() -> bool:
    return _built()


def gemv_splitk_supported(bitwidth, bitwidth2, group_size, N, K, M, residual_rank: int = 0) -> bool:
    r = int(residual_rank or 0)
    return (gemv_stream_supported(bitwidth, bitwidth2, group_size, N, K, M)
            and 0 <= r <= GEMV_SPLITK_MAX_RESIDUAL_RANK and r % 8 == 0)


def gemv_splitk_fht_supported(bitwidth, bitwidth2, group_size, N, K, M, residual_rank: int = 0) -> bool:
    return gemv_splitk_supported(bitwidth, bitwidth2, group_size, N, K, M, residual_rank) and int(K) <= 65536


def gemv_multi_available() -> bool:
    return _built()


def gemv_multi_supported(K, tiles_total, specs, fht: bool = False) -> bool:
    """specs: one (bitwidth, bitwidth2, group_size) per segment, as the reference passes them."""
    specs = list(specs)
    return (_built() and 1 <= len(specs) <= 8 and int(tiles_total) > 0 and int(K) % 64 == 0
            and all(_shape_ok(b1, b2, gs, 128, K) for b1, b2, gs in specs))


def gemv_mlp_available() -> bool:
    return _built()


def gemv_mlp_supported(K, N, specs, fht: bool = False, folds_differ: bool = False) -> bool:
    """With folds_differ (gate and up rotated by different folds) the pair is served only where
    one launch can rotate per segment: 4-bit single-stream segments, group size >= 32, K made of
    at most 8 power-of-two pieces (qgemm_gemv_mlp then leaves gate | up side by side and runs one
    SiLU*mul pass)."""
    specs = list(specs)
    ok = _built() and len(specs) == 2 and all(_shape_ok(b1, b2, gs, N, K) for b1, b2, gs in specs)
    if ok and folds_differ:
        ok = all(int(b1) == 4 and not int(b2 or 0) and int(gs) >= 32 for b1, b2, gs in specs) \
            and bin(int(K)).count("1") <= 8
    return ok


def gemv_split_hint(N: int, K: int) -> int:
    """K-split factor of the tile x split decode kernel for an [N, K] projection (the reference's
    gemv_pick_split mirror, :621-640, re-derived for this device by the library)."""
    return _lib.gemv_pick_split(int(N) // 128, int(K))


# ---- converted-code cache ------------------------------------------------------------------------
_slabs = {}      # (device index, address, bytes, bits, K) -> (slab tensor, keep-alive of the blob or None)
_modules = {}    # operand addresses of one projection -> PalettizedLinear


def forget() -> None:
    """Drop every cached slab copy and module (after blobs were freed or rewritten in place)."""
    _slabs.clear()
    _modules.clear()


class _Raw:
    """A device buffer known only by address: enough of the array interface for torch to view it."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(address), False),
                                         "version": 2}


def _view(address: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_Raw(address, nbytes), device=device)


def _slab_of(address: int, N: int, K: int, bits: int, device, keep=None) -> torch.Tensor:
    nbytes = _lib.packed_bytes(N, K, bits)
    key = (torch.device(device).index, int(address), nbytes, bits, K)
    hit = _slabs.get(key)
    if hit is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().b200lut_repack_from_idxn(int(address), out.data_ptr(), N, K, bits,
                                                           torch.cuda.current_stream(device).cuda_stream))
        hit = (out, keep)
        _slabs[key] = hit
    return hit[0]


def _check_a(A: torch.Tensor, what: str) -> None:
    if not (A.is_cuda and A.dim() == 2 and A.dtype in (torch.float16, torch.bfloat16)):
        raise ValueError(f"{what}: A must be a 2-D CUDA fp16 or bf16 tensor, got {tuple(A.shape)} {A.dtype} on {A.device}")


def _rows_of(indices: torch.Tensor, K: int, bits: int, what: str) -> int:
    per_row = K * bits // 8
    if K % 64 or per_row == 0 or indices.numel() % per_row or (indices.numel() // per_row) % 128:
        raise ValueError(f"{what}: {indices.numel()} index bytes do not form an idx{bits} blob of N x {K} "
                         f"with N % 128 == 0 and K % 64 == 0")
    return indices.numel() // per_row


def _module(A, indices, lut, bitwidth, group_size, indices2, lut2, bitwidth2, resB, resA, bias,
            rot_signs, awq_scale, what):
    """The cached module that serves one set of operands (arguments absent in the reference's
    calls are None or empty tensors there; both are accepted)."""
    def opt(t):
        return None if t is None or (torch.is_tensor(t) and t.numel() == 0) else t
    indices2, lut2, resB, resA, bias = opt(indices2), opt(lut2), opt(resB), opt(resA), opt(bias)
    rot_signs, awq_scale = opt(rot_signs), opt(awq_scale)
    _check_a(A, what)
    K, b1 = A.shape[1], int(bitwidth)
    b2 = int(bitwidth2) if (bitwidth2 and indices2 is not None) else 0
    if (indices2 is None) != (lut2 is None) or (resA is None) != (resB is None):
        raise ValueError(f"{what}: a second stream needs indices2 AND lut2, a residual resA AND resB")
    if lut.dtype != A.dtype:
        raise ValueError(f"{what}: A is {A.dtype} but the LUT is {lut.dtype}; the kernels compute in the LUT dtype")
    if not indices.is_cuda:
        raise ValueError(f"{what}: indices must be a CUDA tensor")
    N = _rows_of(indices, K, b1, what)
    key = (A.device.index, indices.data_ptr(), lut.data_ptr(), b1, int(group_size), N, K,
           0 if indices2 is None else indices2.data_ptr(), 0 if lut2 is None else lut2.data_ptr(), b2,
           0 if resA is None else resA.data_ptr(), 0 if resB is None else resB.data_ptr(),
           0 if bias is None else bias.data_ptr(),
           0 if rot_signs is None else rot_signs.data_ptr(), 0 if awq_scale is None else awq_scale.data_ptr())
    mod = _modules.get(key)
    if mod is None:
        flat = indices.contiguous().view(torch.uint8).reshape(-1)
        if flat.data_ptr() % 16:          # the reference clones misaligned views as well
            flat = flat.clone()
        packed = _slab_of(flat.data_ptr(), N, K, b1, A.device, keep=flat)
        mod = PalettizedLinear.from_packed(packed, lut, b1, int(group_size), N, K, bias=bias)
        if indices2 is not None:
            if _rows_of(indices2, K, b2, what) != N:
                raise ValueError(f"{what}: the two streams describe different N")
            flat2 = indices2.contiguous().view(torch.uint8).reshape(-1)
            if flat2.data_ptr() % 16:
                flat2 = flat2.clone()
            mod._packed2 = _slab_of(flat2.data_ptr(), N, K, b2, A.device, keep=flat2)
            mod.indices2 = torch.empty(0, dtype=torch.uint8, device=A.device)
            mod.lut2 = PalettizedLinear._lut2d(lut2, b2)
            mod.bitwidth2 = b2
        if resA is not None:
            if resA.shape != (N, resB.shape[0]) or resB.shape[1] != K:
                raise ValueError(f"{what}: residual factors {tuple(resA.shape)} / {tuple(resB.shape)} do not fit N={N}, K={K}")
            mod.resA, mod.resB = resA, resB
        if rot_signs is not None:
            if rot_signs.numel() != K:
                raise ValueError(f"{what}: rot_signs must hold K = {K} entries")
            mod.rot_signs = rot_signs.detach().float()
            mod.rotation_k = K
            if awq_scale is not None:
                mod.awq_scale = awq_scale.detach().float()
                mod.fold_order = "rotate_then_awq"
        elif awq_scale is not None:
            raise ValueError(f"{what}: awq_scale without rot_signs")
        _modules[key] = mod
    return mod


# ---- projections that take tensors ------------------------------------------------------------------
def qgemm_per_group_lut(A, indices, lut, bitwidth: int = 4, group_size: int = 32, backend: str = "auto",
                        indices_layout: str = "idx4") -> torch.Tensor:
    """Y = A @ W^T, W palettized (reference :138-187). Any M: decode kernel up to 16 rows, the
    tensor-core GEMM above. `backend` is accepted for compatibility ("auto" / "cutlass_streaming")."""
    if indices_layout not in _LAYOUT_BITS:
        raise ValueError(f"indices_layout={indices_layout!r} is not one of {sorted(_LAYOUT_BITS)}")
    if _LAYOUT_BITS[indices_layout] != int(bitwidth):
        raise ValueError(f"indices_layout={indices_layout!r} means {_LAYOUT_BITS[indices_layout]} bits, "
                         f"but bitwidth={bitwidth}")
    if backend not in ("auto", "cutlass_streaming"):
        raise ValueError(f"backend {backend!r}: this library has one palettized backend (use 'auto')")
    mod = _module(A, indices, lut, bitwidth, group_size, None, None, 0, None, None, None, None, None,
                  "qgemm_per_group_lut")
    return mod(A)


def qgemm_dense(A, W_dense, group_size: int = 32, backend: str = "cutlass_dense") -> torch.Tensor:
    """Dense baseline Y = A @ W_dense^T (reference :190-220): a library GEMM, for benchmarks only."""
    if backend != "cutlass_dense":
        raise ValueError("qgemm_dense only supports backend='cutlass_dense'")
    return torch.matmul(A, W_dense.t())


def qgemm_dual_stream(A, indices, lut, bitwidth, group_size, indices2=None, lut2=None, bitwidth2: int = 0,
                      resB=None, resA=None, bias=None) -> torch.Tensor:
    """C = A @ W1^T (+ A @ W2^T) + (A @ resB^T) @ resA^T + bias in one decode launch, M <= 16
    (reference :271-333)."""
    if A.dim() == 2 and A.shape[0] > DUAL_STREAM_MAX_M:
        raise ValueError(f"qgemm_dual_stream serves M <= {DUAL_STREAM_MAX_M}, got M={A.shape[0]}")
    return _module(A, indices, lut, bitwidth, group_size, indices2, lut2, bitwidth2, resB, resA, bias,
                   None, None, "qgemm_dual_stream")(A)


def _gemv(what, A, indices, lut, bitwidth, group_size, indices2, lut2, bitwidth2, resB, resA, bias,
          rot_signs, awq_scale):
    if A.dim() == 2 and A.shape[0] != 1:
        raise ValueError(f"{what}: the decode GEMV entries of the reference take one row (M == 1), got M={A.shape[0]}")
    return _module(A, indices, lut, bitwidth, group_size, indices2, lut2, bitwidth2, resB, resA, bias,
                   rot_signs, awq_scale, what)(A)


def qgemm_gemv_stream(A, indices, lut, bitwidth, group_size, indices2=None, lut2=None, bitwidth2: int = 0,
                      resB=None, resA=None, bias=None, rot_signs=None, awq_scale=None) -> torch.Tensor:
    """The M == 1 decode GEMV (reference :428-590). With rot_signs, A is the UNROTATED row."""
    return _gemv("qgemm_gemv_stream", A, indices, lut, bitwidth, group_size, indices2, lut2, bitwidth2,
                 resB, resA, bias, rot_signs, awq_scale)


def qgemm_gemv_splitk_stream(A, indices, lut, bitwidth, group_size, indices2=None, lut2=None,
                             bitwidth2: int = 0, resB=None, resA=None, bias=None, rot_signs=None,
                             awq_scale=None) -> torch.Tensor:
    """The M == 1 split-K decode GEMV (reference :734-870); the split is the library's policy."""
    return _gemv("qgemm_gemv_splitk_stream", A, indices, lut, bitwidth, group_size, indices2, lut2,
                 bitwidth2, resB, resA, bias, rot_signs, awq_scale)


# ---- merged launches described by a table of device addresses ------------------------------------------
_COLS = ("q1", "lut1", "q2", "lut2", "resB", "resA", "bias", "C", "N", "R", "b1", "b2", "gs", "signs", "s")


def _check_table(A, seg_table, count, what):
    if not (torch.is_tensor(seg_table) and seg_table.device.type == "cpu" and seg_table.dtype == torch.int64
            and seg_table.dim() == 2 and seg_table.size(1) == 15):
        raise ValueError(f"{what}: seg_table must be a CPU int64 [count, 15] tensor "
                         f"(columns {', '.join(_COLS)})")
    if count is not None and seg_table.size(0) != count:
        raise ValueError(f"{what}: seg_table must have {count} rows, got {seg_table.size(0)}")
    if not 1 <= seg_table.size(0) <= 8:
        raise ValueError(f"{what}: 1..8 segments per launch, got {seg_table.size(0)}")
    _check_a(A, what)
    if not (A.is_contiguous() and A.shape[0] == 1):
        raise ValueError(f"{what}: A must be a contiguous [1, K] tensor")


def _table_segments(rows, members, x, K, dev, dt, out_override, keep):
    """b200lut_segment array of the table rows `members`; residual projections run on `x`."""
    segs = (_lib.Segment * len(members))()
    for sg, i in zip(segs, members):
        r = rows[i]
        N, b1, b2, gs = r["N"], r["b1"], r["b2"], r["gs"]
        if N <= 0 or N % 128 or not r["q1"] or not r["lut1"]:
            raise ValueError(f"seg_table row {i}: N must be a positive multiple of 128 and q1 / lut1 non-zero")
        sg.packed = _slab_of(r["q1"], N, K, b1, dev).data_ptr()
        sg.lut = r["lut1"]
        if r["q2"]:
            sg.packed2 = _slab_of(r["q2"], N, K, b2, dev).data_ptr()
            sg.lut2, sg.bits2 = r["lut2"], b2
        sg.bias = r["bias"] or None
        out = r["C"]
        if out_override is not None:
            out = out_override.get(i, 0)
        sg.out = out or None
        sg.ldo, sg.N, sg.group_size, sg.n_groups, sg.bits = N, N, gs, -(-N // gs), b1
        if r["R"]:
            R = r["R"]
            resB = _view(r["resB"], R * K * 2, dev).view(dt).view(R, K)
            t = _lib.residual_project(x, resB, flags=_flags())
            keep.append(t)
            sg.resA, sg.res_t, sg.res_rank, sg.res_ldt = r["resA"], t.data_ptr(), R, t.stride(0)
    return segs


def _table_launch(A, seg_table, epilogue, out_override=None):
    """Run the segments of a [count, 15] address table. Segments that share one fold (signs, s) —
    or carry none — run as ONE launch on the (rotated) row. Different folds also run as one
    launch where the row-range kernel can rotate per segment (4-bit single-stream segments,
    group size >= 32, no low-rank residual, K of at most 8 power-of-two pieces), as the
    reference does; otherwise one launch per fold, each behind its own transform. Under the
    SiLU*mul epilogue gate and up share one input, so different folds there give one launch
    that leaves gate and up side by side and one SiLU*mul pass (two roundings more than the
    reference's fused kernel)."""
    dev, K, dt = A.device, A.shape[1], A.dtype
    rows = [dict(zip(_COLS, (int(v) for v in r))) for r in seg_table.tolist()]
    rotated = [r["signs"] != 0 for r in rows]
    if any(rotated) and not all(rotated):
        raise ValueError("seg_table: rotation signs must be present on every segment or on none")
    folds = {}
    for i, r in enumerate(rows):
        folds.setdefault((r["signs"], r["s"]), []).append(i)
    keep = []
    override = None if out_override is None else {0: out_override}

    def fold_tensors(signs_ptr, s_ptr):
        signs = _view(signs_ptr, 4 * K, dev).view(torch.float32) if signs_ptr else None
        scale = _view(s_ptr, 4 * K, dev).view(torch.float32) if s_ptr else None
        return signs, scale

    per_segment = (len(folds) > 1 and bin(K).count("1") <= 8
                   and all(r["b1"] == 4 and not r["q2"] and r["gs"] >= 32 and not r["R"] for r in rows))
    if per_segment:
        members = list(range(len(rows)))
        silu = epilogue == _lib.EPI_SILU_MUL
        up = None
        if silu:     # gate lands in C, up beside it, then C <- silu(C) * up
            up = torch.empty(1, rows[1]["N"], dtype=dt, device=dev)
            override = {0: out_override, 1: up.data_ptr()}
        segs = _table_segments(rows, members, A, K, dev, dt, override, keep)
        inp = _lib.make_input(seg_folds=[fold_tensors(r["signs"], r["s"]) for r in rows])
        _lib.gemv_input(A, segs, len(members), inp, flags=_flags())
        if silu:
            gate = _view(out_override, 2 * rows[0]["N"], dev).view(dt).view(1, rows[0]["N"])
            _lib.silu_mul(gate, up)
        return
    if epilogue == _lib.EPI_SILU_MUL and len(folds) > 1:
        raise ValueError("qgemm_gemv_mlp: gate and up with different rotation folds are served for 4-bit "
                         "single-stream segments without a low-rank residual only")
    for (signs_ptr, s_ptr), members in folds.items():
        x = A
        if signs_ptr:
            signs, scale = fold_tensors(signs_ptr, s_ptr)
            x = _lib.fht(A, signs, mode=_lib.FHT_AWQ, scale=scale) if scale is not None else _lib.fht(A, signs)
        segs = _table_segments(rows, members, x, K, dev, dt, override, keep)
        _lib.gemv_multi(x, segs, len(members), epilogue=epilogue, flags=_flags())


def qgemm_gemv_multi(A, seg_table) -> None:
    """1-8 projections that share one input row in one decode launch; the results land in the
    buffers the table's C column names (reference :958-1003). Table columns: q1, lut1, q2, lut2,
    resB, resA, bias, C, N, R, b1, b2, gs, signs, s as raw device addresses / integers, 0 = not
    supplied. Every LUT holds ceil(N / gs) palette rows."""
    _check_table(A, seg_table, None, "qgemm_gemv_multi")
    _table_launch(A, seg_table, _lib.EPI_NONE)


def qgemm_gemv_mlp(A, seg_table, C) -> torch.Tensor:
    """C = silu(gate(A)) * up(A): row 0 of the table is the gate projection, row 1 the up
    projection; one launch, one rounding (reference :1057-1109). Returns C."""
    _check_table(A, seg_table, 2, "qgemm_gemv_mlp")
    if int(seg_table[0, 8]) != int(seg_table[1, 8]):
        raise ValueError("qgemm_gemv_mlp: gate and up must have the same N")
    if not (torch.is_tensor(C) and C.is_cuda and C.dtype == A.dtype and C.numel() == int(seg_table[0, 8])
            and C.is_contiguous()):
        raise ValueError("qgemm_gemv_mlp: C must be a contiguous CUDA [1, N] tensor of A's dtype")
    _table_launch(A, seg_table, _lib.EPI_SILU_MUL, out_override=C.data_ptr())
    return C
