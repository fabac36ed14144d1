"""ctypes binding of libb200lut.so (the C ABI declared in include/b200_lut.h).

The library is the only compute path of this package: if it is missing or a
call fails, an exception is raised — nothing falls back to torch or the CPU.
Tensors are passed as raw device pointers; launches go to torch's current CUDA
stream so they order with the surrounding torch work.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200lut.so")

OK = 0
BF16, F16, F32 = 0, 1, 2
EPI_NONE, EPI_SILU_MUL = 0, 1
FHT_FORWARD, FHT_ADJOINT, FHT_AWQ = 0, 1, 2
FLAG_PDL = 1
FLAG_TILE_KERNEL = 2     # decode GEMV: force the tile x K-split kernel
FLAG_ROWS_KERNEL = 4     # decode GEMV: the row-range kernel where it serves the shapes
FLAG_CTA_PAIRS = 8       # prefill GEMM: CTA pairs (tcgen05 cta_group::2); slower, never the default

EXPORTS = (
    "b200lut_version", "b200lut_last_error", "b200lut_sm_count", "b200lut_device_status", "b200lut_packed_bytes",
    "b200lut_repack_from_idxn", "b200lut_repack_to_idxn", "b200lut_unpack_codes",
    "b200lut_dequant", "b200lut_gemv_workspace_bytes", "b200lut_gemv_pick_split",
    "b200lut_gemv_multi", "b200lut_gemv", "b200lut_gemm", "b200lut_fht",
    "b200lut_residual_project", "b200lut_residual_project_rows", "b200lut_silu_mul", "b200lut_gemm_workspace_bytes", "b200lut_gemm_ws", "b200lut_gemm_multi",
    "b200lut_gemm_two_stream", "b200lut_gemm_two_stream_bytes",
    "b200lut_embed_gather", "b200lut_round_rows", "b200lut_gemv_kgrouped",
    "b200lut_gemv_kgrouped_split", "b200lut_gemv_kgrouped_workspace_bytes", "b200lut_gemm_kgrouped", "b200lut_gemv_exchange", "b200lut_peer_export", "b200lut_peer_open", "b200lut_peer_close",
    "b200lut_gemv_noalloc", "b200lut_gemv_noalloc_reset", "b200lut_gemv_launch_blocks", "b200lut_gemv_input", "b200lut_plan_bytes", "b200lut_plan_build", "b200lut_plan_run", "b200lut_plan_status", "b200lut_plan_form", "b200lut_plan_release",
)


class Segment(ctypes.Structure):
    """struct b200lut_segment."""
    _fields_ = [
        ("packed", ctypes.c_void_p), ("lut", ctypes.c_void_p),
        ("packed2", ctypes.c_void_p), ("lut2", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("ldo", ctypes.c_int64),
        ("N", ctypes.c_int), ("group_size", ctypes.c_int), ("n_groups", ctypes.c_int),
        ("bits", ctypes.c_int), ("bits2", ctypes.c_int), ("res_rank", ctypes.c_int),
        ("resA", ctypes.c_void_p), ("res_t", ctypes.c_void_p), ("res_ldt", ctypes.c_int64),
    ]


class Job(ctypes.Structure):
    """struct b200lut_job."""
    _fields_ = [
        ("x", ctypes.c_void_p), ("ldx", ctypes.c_int64),
        ("K", ctypes.c_int), ("nseg", ctypes.c_int), ("epilogue", ctypes.c_int),
        ("dep", ctypes.c_int), ("segs", Segment * 8),
    ]


MAX_PEERS = 8


class Exchange(ctypes.Structure):
    """struct b200lut_exchange."""
    _fields_ = [
        ("world", ctypes.c_int), ("rank", ctypes.c_int),
        ("push", ctypes.c_int), ("wait", ctypes.c_int),
        ("producer_blocks", ctypes.c_int), ("wait_ms", ctypes.c_int),
        ("peer_delta", ctypes.c_int64 * MAX_PEERS), ("peer_flag", ctypes.c_void_p * MAX_PEERS),
        ("ticket", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("flags", ctypes.c_void_p),
        ("wait_ticket", ctypes.c_void_p), ("wait_count", ctypes.c_void_p),
        ("sentinel", ctypes.c_int), ("reserved", ctypes.c_int),
    ]


class Input(ctypes.Structure):
    """struct b200lut_input: what a decode launch does to its activation rows first."""
    _fields_ = [("x_mul", ctypes.c_void_p), ("rot_signs", ctypes.c_void_p), ("awq_scale", ctypes.c_void_p),
                ("per_segment", ctypes.c_int), ("seg_rot_signs", ctypes.c_void_p * 8),
                ("seg_awq_scale", ctypes.c_void_p * 8)]


class LibraryError(RuntimeError):
    """A b200lut_* call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b200lut status {code}: {message}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once; loud failure when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
            "(nvcc, sm_100a). This package has no other compute path.")
    L = ctypes.CDLL(LIB_PATH)
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
    L.b200lut_version.restype = i32
    L.b200lut_last_error.restype = ctypes.c_char_p
    L.b200lut_sm_count.restype = i32
    L.b200lut_device_status.restype = i32
    L.b200lut_packed_bytes.restype = sz
    L.b200lut_packed_bytes.argtypes = [i32, i32, i32]
    for name in ("b200lut_repack_from_idxn", "b200lut_repack_to_idxn", "b200lut_unpack_codes"):
        getattr(L, name).restype = i32
        getattr(L, name).argtypes = [vp, vp, i32, i32, i32, vp]
    L.b200lut_dequant.restype = i32
    L.b200lut_dequant.argtypes = [vp, vp, i32, vp, i32, i32, i32, i32, vp]
    L.b200lut_gemv_workspace_bytes.restype = sz
    L.b200lut_gemv_workspace_bytes.argtypes = [i32, i32, i32]
    L.b200lut_gemv_pick_split.restype = i32
    L.b200lut_gemv_pick_split.argtypes = [i32, i32]
    L.b200lut_gemv_multi.restype = i32
    L.b200lut_gemv_multi.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, i32,
                                     i32, vp, sz, i32, vp]
    L.b200lut_gemm_workspace_bytes.restype = sz
    L.b200lut_gemm_workspace_bytes.argtypes = [i32, i32, i32]
    L.b200lut_gemm_ws.restype = i32
    L.b200lut_gemm_ws.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, i32, vp, sz, vp]
    L.b200lut_gemm_multi.restype = i32
    L.b200lut_gemm_multi.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, i32, vp, sz, vp]
    L.b200lut_gemv_kgrouped_split.restype = i32
    L.b200lut_gemv_kgrouped_split.argtypes = [i32, i32]
    L.b200lut_gemv_kgrouped_workspace_bytes.restype = sz
    L.b200lut_gemv_kgrouped_workspace_bytes.argtypes = [i32, i32, i32]
    L.b200lut_gemv_kgrouped.restype = i32
    L.b200lut_gemv_kgrouped.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, i32, i32, vp, i64, i32, vp, sz, vp]
    L.b200lut_gemm_kgrouped.restype = i32
    L.b200lut_gemm_kgrouped.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, i32, i32, vp, i64, i32, vp, sz, vp]
    L.b200lut_gemm_two_stream_bytes.restype = sz
    L.b200lut_gemm_two_stream_bytes.argtypes = [i32, i32]
    L.b200lut_gemm_two_stream.restype = i32
    L.b200lut_gemm_two_stream.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, vp, sz, vp]
    L.b200lut_embed_gather.restype = i32
    L.b200lut_embed_gather.argtypes = [vp, i64, i32, i32, ctypes.POINTER(Segment), vp, i32, vp]
    L.b200lut_round_rows.restype = i32
    L.b200lut_round_rows.argtypes = [vp, i64, vp, i64, i64, i32, i32, vp]
    L.b200lut_silu_mul.restype = i32
    L.b200lut_silu_mul.argtypes = [vp, vp, i32, i32, i64, i64, i32, vp]
    L.b200lut_residual_project.restype = i32
    L.b200lut_residual_project.argtypes = [vp, i64, i32, i32, i32, vp, i32, vp, i64, i32, vp]
    L.b200lut_residual_project_rows.restype = i32
    L.b200lut_residual_project_rows.argtypes = [vp, i64, i32, i32, i32, vp, i32, vp, i64, i32, i32, vp]
    L.b200lut_gemv_exchange.restype = i32
    L.b200lut_gemv_exchange.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, i32,
                                        i32, vp, sz, i32, ctypes.POINTER(Exchange), vp]
    L.b200lut_peer_export.restype = i32
    L.b200lut_peer_export.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(i64)]
    L.b200lut_peer_open.restype = i32
    L.b200lut_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.b200lut_peer_close.restype = i32
    L.b200lut_peer_close.argtypes = [vp]
    L.b200lut_gemv.restype = i32
    L.b200lut_gemv.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, sz, vp]
    L.b200lut_gemm.restype = i32
    L.b200lut_gemm.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, i32, vp]
    L.b200lut_fht.restype = i32
    L.b200lut_fht.argtypes = [vp, vp, vp, vp, i32, i32, i64, i64, i32, i32, i32, vp]
    L.b200lut_gemv_noalloc.restype = i32
    L.b200lut_gemv_noalloc.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]
    L.b200lut_gemv_input.restype = i32
    L.b200lut_gemv_input.argtypes = [vp, i64, i32, i32, i32, ctypes.POINTER(Segment), i32, i32,
                                     i32, vp, sz, i32, ctypes.POINTER(Exchange), ctypes.POINTER(Input), vp]
    L.b200lut_gemv_launch_blocks.restype = i32
    L.b200lut_gemv_launch_blocks.argtypes = [i32, i32, ctypes.POINTER(Segment), i32, i32, i32]
    L.b200lut_gemv_noalloc_reset.restype = i32
    L.b200lut_gemv_noalloc_reset.argtypes = [vp]
    L.b200lut_plan_bytes.restype = sz
    L.b200lut_plan_bytes.argtypes = [ctypes.POINTER(Job), i32, i32, i32]
    L.b200lut_plan_build.restype = i32
    L.b200lut_plan_build.argtypes = [vp, sz, ctypes.POINTER(Job), i32, i32, i32, vp]
    L.b200lut_plan_run.restype = i32
    L.b200lut_plan_run.argtypes = [vp, i32, i32, vp]
    L.b200lut_plan_status.restype = i32
    L.b200lut_plan_status.argtypes = [vp]
    L.b200lut_plan_form.restype = i32
    L.b200lut_plan_form.argtypes = [vp]
    L.b200lut_plan_release.restype = i32
    L.b200lut_plan_release.argtypes = [vp]
    _lib = L
    return L


def check(code: int) -> None:
    if code != OK:
        raise LibraryError(code, lib().b200lut_last_error().decode("utf-8", "replace"))


def dtype_id(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float16:
        return F16
    if dtype == torch.float32:
        return F32
    raise TypeError(f"unsupported dtype {dtype}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: this package computes on the GPU only")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------- #
# layout
# --------------------------------------------------------------------------- #

def packed_bytes(N: int, K: int, bits: int) -> int:
    n = lib().b200lut_packed_bytes(N, K, bits)
    if n == 0:
        raise ValueError(f"idxN layout requires N%128==0 and K%64==0 and bits in 1..4, got "
                         f"N={N}, K={K}, bits={bits}")
    return n


def repack_from_idxn(blob: torch.Tensor, N: int, K: int, bits: int) -> torch.Tensor:
    """idxN blob (uint8, CUDA) -> slab-layout codes (uint8, CUDA)."""
    _need_cuda(blob, "blob")
    blob = blob.contiguous().view(torch.uint8).reshape(-1)
    n = packed_bytes(N, K, bits)
    if blob.numel() != n:
        raise ValueError(f"idx{bits} blob numel {blob.numel()} != N*K*{bits}/8 {n} (N={N}, K={K})")
    if blob.data_ptr() % 16:
        blob = blob.clone()
    out = torch.empty(n, dtype=torch.uint8, device=blob.device)
    with torch.cuda.device(blob.device):
        check(lib().b200lut_repack_from_idxn(blob.data_ptr(), out.data_ptr(), N, K, bits, _stream(blob)))
    return out


def repack_to_idxn(packed: torch.Tensor, N: int, K: int, bits: int) -> torch.Tensor:
    _need_cuda(packed, "packed")
    out = torch.empty(packed_bytes(N, K, bits), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().b200lut_repack_to_idxn(packed.data_ptr(), out.data_ptr(), N, K, bits, _stream(packed)))
    return out


def unpack_codes(packed: torch.Tensor, N: int, K: int, bits: int) -> torch.Tensor:
    _need_cuda(packed, "packed")
    out = torch.empty(N, K, dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().b200lut_unpack_codes(packed.data_ptr(), out.data_ptr(), N, K, bits, _stream(packed)))
    return out


def dequant(packed: torch.Tensor, lut: torch.Tensor, N: int, K: int, bits: int,
            group_size: int) -> torch.Tensor:
    """[N, K] tensor of the palette entries (dtype of the LUT, exact)."""
    _need_cuda(packed, "packed")
    lut = lut.contiguous()
    if lut.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"LUT dtype must be bfloat16 or float16, got {lut.dtype}")
    out = torch.empty(N, K, dtype=lut.dtype, device=packed.device)
    n_groups = lut.numel() >> bits
    with torch.cuda.device(packed.device):
        check(lib().b200lut_dequant(packed.data_ptr(), lut.data_ptr(), n_groups, out.data_ptr(),
                                    N, K, bits, group_size, _stream(packed)))
    return out


# --------------------------------------------------------------------------- #
# compute
# --------------------------------------------------------------------------- #

def make_segments(descs: Sequence[dict]):
    """Build a ctypes array of b200lut_segment from dicts of tensors/ints."""
    arr = (Segment * len(descs))()
    for s, d in zip(arr, descs):
        s.packed, s.lut = ptr(d["packed"]), ptr(d["lut"])
        s.packed2, s.lut2 = ptr(d.get("packed2")), ptr(d.get("lut2"))
        s.bias, s.out = ptr(d.get("bias")), ptr(d.get("out"))
        s.ldo = int(d.get("ldo", d["N"]))
        s.N, s.group_size, s.n_groups = int(d["N"]), int(d["group_size"]), int(d["n_groups"])
        s.bits, s.bits2 = int(d["bits"]), int(d.get("bits2") or 0)
        if d.get("resA") is not None:
            t = d["res_t"]
            s.resA, s.res_t = ptr(d["resA"]), t.data_ptr()
            s.res_rank, s.res_ldt = int(d["resA"].shape[1]), int(t.stride(0))
    return arr


def residual_project(x: torch.Tensor, resB: torch.Tensor, flags: int = 0,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """t = x @ resB^T in fp32 ([M, R]); the first factor of the fused low-rank residual."""
    _need_cuda(x, "x")
    M, K = x.shape
    R = resB.shape[0]
    if out is None:
        out = torch.empty(M, R, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().b200lut_residual_project(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype),
                                             resB.data_ptr(), R, out.data_ptr(), out.stride(0),
                                             flags, _stream(x)))
    return out


def residual_block_cols(rank: int) -> int:
    """Columns of a projection's block of the prefill t matrix: 64 * ceil(rank / 64)."""
    return 64 * ((int(rank) + 63) // 64)


def residual_project_rows(x: torch.Tensor, resB: torch.Tensor, flags: int = 0,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """t = round(x @ resB^T) in x's dtype for the prefill GEMM: [M, 64 * ceil(R / 64)], zero
    beyond column R. `out` may be a column block of a wider matrix (merged launches)."""
    _need_cuda(x, "x")
    M, K = x.shape
    R = resB.shape[0]
    cols = residual_block_cols(R)
    if out is None:
        out = torch.empty(M, cols, dtype=x.dtype, device=x.device)
    if out.shape[1] != cols or out.dtype != x.dtype or out.stride(1) != 1:
        raise ValueError("residual_project_rows: out must be [M, 64 * ceil(R / 64)] in x's dtype")
    with torch.cuda.device(x.device):
        check(lib().b200lut_residual_project_rows(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype),
                                                  resB.data_ptr(), R, out.data_ptr(), out.stride(0),
                                                  cols, flags, _stream(x)))
    return out


def gemv_workspace_bytes(total_rows: int, M: int, split: int) -> int:
    return lib().b200lut_gemv_workspace_bytes(total_rows, M, split)


def gemv_multi(x: torch.Tensor, segs, nseg: int, epilogue: int = EPI_NONE, split: int = 0,
               workspace: Optional[torch.Tensor] = None, flags: int = 0) -> None:
    """Launch the decode GEMV over a prepared segment array (outputs are the
    tensors whose pointers the segments carry)."""
    _need_cuda(x, "x")
    M, K = x.shape
    ws_ptr = None if workspace is None else workspace.data_ptr()
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    with torch.cuda.device(x.device):
        check(lib().b200lut_gemv_multi(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), segs,
                                       nseg, epilogue, split, ws_ptr, ws_bytes, flags, _stream(x)))


def gemv_launch_blocks(M: int, K: int, segs, nseg: int, epilogue: int = EPI_NONE, flags: int = 0) -> int:
    """Blocks of the launch gemv_multi / gemv_exchange would make with split = 0."""
    n = int(lib().b200lut_gemv_launch_blocks(M, K, segs, nseg, epilogue, flags))
    if n <= 0:
        raise ValueError("gemv_launch_blocks: invalid launch description")
    return n


def gemv_pick_split(tiles: int, K: int) -> int:
    return int(lib().b200lut_gemv_pick_split(tiles, K))


def gemv_exchange(x: torch.Tensor, segs, nseg: int, ex: "Exchange", epilogue: int = EPI_NONE,
                  split: int = 0, flags: int = 0) -> None:
    """gemv_multi with the column-parallel exchange folded in (push after, wait before)."""
    _need_cuda(x, "x")
    M, K = x.shape
    with torch.cuda.device(x.device):
        check(lib().b200lut_gemv_exchange(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), segs,
                                          nseg, epilogue, split, None, 0, flags,
                                          ctypes.byref(ex), _stream(x)))


def make_input(x_mul: Optional[torch.Tensor] = None, rot_signs: Optional[torch.Tensor] = None,
               awq_scale: Optional[torch.Tensor] = None, seg_folds=None) -> Input:
    """An input transform for gemv_input (tensors must stay alive while it is used).
    seg_folds: one (rot_signs or None, awq_scale or None) pair per segment of the launch — every
    segment rotates the shared rows with its own fold (excludes rot_signs / awq_scale)."""
    folds = list(seg_folds) if seg_folds is not None else []
    if folds and (rot_signs is not None or awq_scale is not None):
        raise ValueError("per-segment folds exclude a launch-wide fold")
    if len(folds) > 8:
        raise ValueError("at most 8 segments per launch")
    flat = [("rot_signs", rot_signs), ("awq_scale", awq_scale)]
    flat += [(f"seg_folds[{i}]", v) for i, pair in enumerate(folds) for v in pair]
    for name, v in flat:
        if v is not None and (v.dtype != torch.float32 or not v.is_contiguous() or not v.is_cuda):
            raise ValueError(f"{name} must be a contiguous float32 CUDA tensor")
    inp = Input()
    inp.x_mul, inp.rot_signs, inp.awq_scale = ptr(x_mul), ptr(rot_signs), ptr(awq_scale)
    if folds:
        inp.per_segment = 1
        for i, (sg, aw) in enumerate(folds):
            inp.seg_rot_signs[i], inp.seg_awq_scale[i] = ptr(sg), ptr(aw)
    return inp


def gemv_input(x: torch.Tensor, segs, nseg: int, inp: Input, epilogue: int = EPI_NONE, flags: int = 0,
               ex: Optional["Exchange"] = None) -> None:
    """gemv_multi whose launch first transforms the activation rows (silu(x) * x_mul, Hadamard
    rotation); raises LibraryError (code 2) when the shapes are not served in fused form."""
    _need_cuda(x, "x")
    M, K = x.shape
    with torch.cuda.device(x.device):
        check(lib().b200lut_gemv_input(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), segs, nseg,
                                       epilogue, 0, None, 0, flags,
                                       None if ex is None else ctypes.byref(ex), ctypes.byref(inp), _stream(x)))


def peer_export(t: torch.Tensor):
    """(64-byte handle, offset) of the device allocation that holds tensor t."""
    _need_cuda(t, "buffer")
    handle = ctypes.create_string_buffer(64)
    off = ctypes.c_int64(0)
    with torch.cuda.device(t.device):
        check(lib().b200lut_peer_export(t.data_ptr(), handle, ctypes.byref(off)))
    return bytes(handle.raw), int(off.value)


def peer_open(handle: bytes) -> int:
    base = ctypes.c_void_p(0)
    check(lib().b200lut_peer_open(ctypes.c_char_p(handle), ctypes.byref(base)))
    return int(base.value)


def peer_close(base: int) -> None:
    check(lib().b200lut_peer_close(ctypes.c_void_p(base)))


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """gate <- silu(gate) * up, in place (2-D, last dim contiguous, 16-bit)."""
    _need_cuda(gate, "gate")
    M, N = gate.shape
    with torch.cuda.device(gate.device):
        check(lib().b200lut_silu_mul(gate.data_ptr(), up.data_ptr(), M, N, gate.stride(0), up.stride(0),
                                     dtype_id(gate.dtype), _stream(gate)))
    return gate


def embed_gather(ids: torch.Tensor, table: dict, K: int, dtype: torch.dtype,
                 out_fp32: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ids (1-D int64 CUDA tensor) of a palettized [N, K] table -> [n, K] in `dtype`
    (fp32 with out_fp32). table: packed, lut, bits, N, group_size, n_groups and optionally
    packed2 / lut2 / bits2 and resA + resB (both or neither). out: a contiguous [n, K] tensor of
    the result type to write into (nothing is allocated then)."""
    _need_cuda(ids, "ids")
    if ids.dim() != 1 or ids.dtype != torch.int64 or not ids.is_contiguous():
        raise ValueError("embed_gather expects a contiguous 1-D int64 id tensor")
    n = ids.numel()
    want = torch.float32 if out_fp32 else dtype
    if out is None:
        out = torch.empty(n, K, dtype=want, device=ids.device)
    elif (tuple(out.shape) != (n, K) or out.dtype != want or not out.is_contiguous()
          or out.device != ids.device):
        raise ValueError(f"out must be a contiguous [{n}, {K}] {want} tensor on the ids' device")
    seg = (Segment * 1)()
    s = seg[0]
    s.packed, s.lut = ptr(table["packed"]), ptr(table["lut"])
    s.packed2, s.lut2 = ptr(table.get("packed2")), ptr(table.get("lut2"))
    s.out, s.ldo = out.data_ptr(), K
    s.N, s.group_size, s.n_groups = int(table["N"]), int(table["group_size"]), int(table["n_groups"])
    s.bits, s.bits2 = int(table["bits"]), int(table.get("bits2") or 0)
    resA, resB = table.get("resA"), table.get("resB")
    if resA is not None:
        s.resA, s.res_rank = ptr(resA), int(resA.shape[1])
    with torch.cuda.device(ids.device):
        check(lib().b200lut_embed_gather(ids.data_ptr(), n, K, dtype_id(dtype), seg, ptr(resB),
                                         1 if out_fp32 else 0, _stream(ids)))
    return out


def round_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """fp32 [M, K] rows -> `dtype` (one rounding)."""
    _need_cuda(x, "x")
    M, K = x.shape
    out = torch.empty(M, K, dtype=dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().b200lut_round_rows(x.data_ptr(), x.stride(0), out.data_ptr(), K, M, K,
                                       dtype_id(dtype), _stream(x)))
    return out


_gemm_scratch = {}


def _gemm_workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Scratch of the prefill GEMM's split schedule, one per device and stream (a buffer serves
    one launch at a time, and launches of one stream are ordered): zero-filled when
    (re)allocated, grown geometrically."""
    key = (device, stream)
    buf = _gemm_scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(nbytes, 2 * buf.numel() if buf is not None else 0)
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _gemm_scratch[key] = buf
    return buf


def gemm(x: torch.Tensor, seg, epilogue: int = EPI_NONE, flags: int = 0, split: bool = True) -> None:
    """Prefill GEMM over one segment; brings the scratch buffer of the split schedule when the
    shape gains from it (split=False: whole-tile schedule)."""
    _need_cuda(x, "x")
    M, K = x.shape
    with torch.cuda.device(x.device):
        s0 = seg[0]
        need = lib().b200lut_gemm_workspace_bytes(M, int(s0.N), K) if (split and not s0.packed2) else 0
        if need:
            ws = _gemm_workspace(x.device, int(_stream(x) or 0), need)
            check(lib().b200lut_gemm_ws(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), seg,
                                        epilogue, flags, ws.data_ptr(), ws.numel(), _stream(x)))
        else:
            check(lib().b200lut_gemm(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), seg,
                                     epilogue, flags, _stream(x)))


_kg_scratch = {}


def gemv_kgrouped(x: torch.Tensor, packed: torch.Tensor, lut_k: torch.Tensor, N: int, bits: int,
                  bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  split: int = 0) -> torch.Tensor:
    """Decode GEMV with K-grouped palettes: x [M <= 16, K], codes in the slab layout,
    lut_k [K / 128, N, 2**bits] in x's dtype -> [M, N]."""
    _need_cuda(x, "x")
    M, K = x.shape
    if out is None:
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        # split = 0 leaves the choice (kernel and split) to the library; the scratch is sized for
        # the split it would pick for its workspace-folded kernel
        planned = split if split > 0 else lib().b200lut_gemv_kgrouped_split(N, K)
        need = lib().b200lut_gemv_kgrouped_workspace_bytes(N, M, planned)
        ws = None
        if need:
            # One zero-filled scratch per (device, stream). The tickets sit at its start, N / 128
            # of them, and the partial sums behind them: a call with MORE row tiles than the last
            # one finds old partial sums where its tickets are, so the head is zeroed again
            # (stream-ordered) whenever the tile count changes.
            key = (x.device, int(_stream(x) or 0))
            ws, tiles = _kg_scratch.get(key, (None, 0))
            if ws is None or ws.numel() < need:
                ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=x.device)
            elif tiles != N // 128:
                ws[:(max(tiles, N // 128) * 4 + 511) // 256 * 256].zero_()
            _kg_scratch[key] = (ws, N // 128)
        check(lib().b200lut_gemv_kgrouped(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype),
                                          packed.data_ptr(), lut_k.data_ptr(), ptr(bias), N, bits,
                                          out.data_ptr(), out.stride(0), split, ptr(ws),
                                          ws.numel() if ws is not None else 0, _stream(x)))
    return out


def gemm_kgrouped(x: torch.Tensor, packed: torch.Tensor, lut_k: torch.Tensor, N: int, bits: int,
                  bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  flags: int = 0, split: bool = True) -> torch.Tensor:
    """Tensor-core GEMM with K-grouped palettes, any M: x [M, K], codes in the slab layout,
    lut_k [K / 128, N, 2**bits] in x's dtype -> [M, N] (split=False: whole-tile schedule)."""
    _need_cuda(x, "x")
    M, K = x.shape
    if out is None:
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        need = lib().b200lut_gemm_workspace_bytes(M, N, K) if split else 0
        ws = _gemm_workspace(x.device, int(_stream(x) or 0), need) if need else None
        check(lib().b200lut_gemm_kgrouped(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype),
                                          packed.data_ptr(), lut_k.data_ptr(), ptr(bias), N, bits,
                                          out.data_ptr(), out.stride(0), flags, ptr(ws),
                                          ws.numel() if ws is not None else 0, _stream(x)))
    return out


def gemm_two_stream(x: torch.Tensor, seg, flags: int = 0) -> None:
    """Prefill GEMM of one projection with two code streams of any widths: two tensor-core
    launches that share fp32 sums through a scratch buffer, one rounding."""
    _need_cuda(x, "x")
    M, K = x.shape
    with torch.cuda.device(x.device):
        need = lib().b200lut_gemm_two_stream_bytes(M, int(seg[0].N))
        key = (x.device, int(_stream(x) or 0), "two")
        buf = _gemm_scratch.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty(max(need, 2 * buf.numel() if buf is not None else 0), dtype=torch.uint8,
                              device=x.device)
            _gemm_scratch[key] = buf
        check(lib().b200lut_gemm_two_stream(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), seg, flags,
                                            buf.data_ptr(), buf.numel(), _stream(x)))


GEMM_MULTI_MAX = 4


def gemm_multi_ok(descs: Sequence[dict], K: int) -> bool:
    """True when the projections described by `descs` (dicts as for make_segments) can run as
    one merged prefill launch: at most four, one code stream each, one code width, one group
    size >= 64, K >= 128."""
    if not 1 <= len(descs) <= GEMM_MULTI_MAX or K < 128:
        return False
    d0 = descs[0]
    return all(d.get("packed2") is None and d["bits"] == d0["bits"]
               and d["group_size"] == d0["group_size"] and d["group_size"] >= 64 for d in descs)


def gemm_multi(x: torch.Tensor, segs, nseg: int, flags: int = 0, split: bool = True) -> None:
    """Prefill GEMM over `nseg` projections that share x, as one launch."""
    _need_cuda(x, "x")
    M, K = x.shape
    with torch.cuda.device(x.device):
        total = sum(int(segs[i].N) for i in range(nseg))
        need = lib().b200lut_gemm_workspace_bytes(M, total, K) if split else 0
        ws = _gemm_workspace(x.device, int(_stream(x) or 0), need) if need else None
        check(lib().b200lut_gemm_multi(x.data_ptr(), x.stride(0), M, K, dtype_id(x.dtype), segs, nseg,
                                       flags, ptr(ws), ws.numel() if ws is not None else 0, _stream(x)))


def fht(x: torch.Tensor, signs: Optional[torch.Tensor], mode: int = FHT_FORWARD,
        scale: Optional[torch.Tensor] = None, block: int = 0,
        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise Hadamard transform of a 2-D CUDA tensor (last dim contiguous)."""
    _need_cuda(x, "x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("fht expects a 2-D tensor with a contiguous last dim")
    M, K = x.shape
    if out is None:
        out = torch.empty(M, K, dtype=x.dtype, device=x.device)
    for name, v in (("signs", signs), ("scale", scale)):
        if v is not None and (v.dtype != torch.float32 or not v.is_contiguous()
                              or v.numel() != K or v.device != x.device):
            raise ValueError(f"{name} must be a contiguous (K,) float32 tensor on x's device")
    with torch.cuda.device(x.device):
        check(lib().b200lut_fht(x.data_ptr(), out.data_ptr(), ptr(signs), ptr(scale), M, K,
                                x.stride(0), out.stride(0), dtype_id(x.dtype), mode, block,
                                _stream(x)))
    return out


class DecodePlan:
    """A persistent decode plan: a list of decode GEMV jobs run by ONE cooperative
    launch (b200lut_plan_*). jobs: dicts with x (CUDA tensor [M, K]), segs (list of
    segment dicts as for make_segments), epilogue and dep (index of the producing job
    or -1). The plan keeps references to every tensor it points to."""

    def __init__(self, jobs: Sequence[dict], M: int, dtype: torch.dtype, device):
        self.M, self.dtype, self.device = int(M), dtype, torch.device(device)
        self._keep = list(jobs)
        arr = (Job * len(jobs))()
        for j, d in zip(arr, jobs):
            x = d["x"]
            _need_cuda(x, "x")
            if x.shape[0] != M or x.stride(1) != 1:
                raise ValueError("every job's x must be [M, K] with a contiguous last dim")
            j.x, j.ldx, j.K = x.data_ptr(), x.stride(0), x.shape[1]
            segs = make_segments(d["segs"])
            j.nseg, j.epilogue, j.dep = len(d["segs"]), int(d.get("epilogue", EPI_NONE)), int(d.get("dep", -1))
            for i in range(len(d["segs"])):
                j.segs[i] = segs[i]
        did = dtype_id(dtype)
        with torch.cuda.device(self.device):
            nbytes = lib().b200lut_plan_bytes(arr, len(jobs), self.M, did)
            if nbytes == 0:
                check(lib().b200lut_plan_build(None, 0, arr, len(jobs), self.M, did, None) or 1)
            self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            check(lib().b200lut_plan_build(self.buffer.data_ptr(), nbytes, arr, len(jobs), self.M, did,
                                           torch.cuda.current_stream(self.device).cuda_stream))
        self.njobs = len(jobs)
        # "rows": the row-range block body runs job after job; "tiles": the tile-share kernel
        self.form = "rows" if lib().b200lut_plan_form(self.buffer.data_ptr()) == 1 else "tiles"

    def run(self) -> None:
        with torch.cuda.device(self.device):
            check(lib().b200lut_plan_run(self.buffer.data_ptr(), self.M, dtype_id(self.dtype),
                                         torch.cuda.current_stream(self.device).cuda_stream))

    def check_status(self) -> None:
        with torch.cuda.device(self.device):
            check(lib().b200lut_plan_status(self.buffer.data_ptr()))

    def close(self) -> None:
        """Drop the library's record of this plan (before its buffer goes back to the allocator)."""
        buf = self.__dict__.get("buffer")
        if buf is not None and _lib is not None:
            with torch.cuda.device(self.device):
                lib().b200lut_plan_release(buf.data_ptr())

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
