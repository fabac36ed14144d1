"""Runtime modules of the LUT-palettized linear layer on B200.

Drop-in for the linear modules of the reference's
src/scripts/palettized_modules.py: PalettizedLinear (:413-1369, same constructor
signature and attribute names), SplitQKV (:1390-1466), FusedPalettizedMLP
(:1643-1723) and reference_dequant (:125-162). Every forward runs on the CUDA
library (libb200lut.so); there is no torch/CPU compute fallback:

  M <= 16  -> b200lut_gemv_multi  (decode GEMV; split-K, merged QKV, fused gate/up)
  M  > 16  -> b200lut_gemm        (prefill GEMM on tcgen05 / TMEM)
  rotation -> b200lut_fht in front of either
  reference=True -> the same arithmetic as the reference's torch route
                    (dequantise exactly, fp32 matmul, one rounding), on the GPU.

Weights: W[n, k] = LUT[min(n // group_size, G-1)][idx[n, k]] — groups run along
the output rows, one palette row serves all of K. The module receives the idxN
blob and converts it once, on the device, into the library's slab layout.
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch
import torch.nn as nn

from . import _lib
from . import fht as _fht
from . import idxN as _idxn

GEMV_MAX_M = 16
# Programmatic dependent launch is ON unless B200LUT_PDL=0: a launch then fetches its codes and
# palettes and builds its tables while the previous kernel of the stream drains, and waits for it
# only before it reads activations. Weights must therefore not be rewritten by the kernel that
# directly precedes a forward in the stream (load-time conversions are followed by the module's
# first forward only after their own kernels have completed their blocks).
_LAUNCH_FLAGS = {"pdl": os.environ.get("B200LUT_PDL", "1").strip() not in ("0", "false", "False")}
_workspaces = {}


def set_programmatic_launch(enabled: bool) -> None:
    """Launch decode kernels with programmatic dependent launch (their weight
    prefetch then overlaps the previous kernel's tail)."""
    _LAUNCH_FLAGS["pdl"] = bool(enabled)


def _flags() -> int:
    return _lib.FLAG_PDL if _LAUNCH_FLAGS["pdl"] else 0


def _workspace(device, nbytes: int) -> Optional[torch.Tensor]:
    """Per-device zero-initialised scratch for splits wider than a cluster."""
    if nbytes == 0:
        return None
    ws = _workspaces.get(str(device))
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[str(device)] = ws
    return ws


def reference_dequant(indices_blob, lut, N: int, K: int, group_size: int,
                      bitwidth: int = 4) -> torch.Tensor:
    """W[n, k] = LUT[n // gs, idx(n, k)] as an (N, K) fp32 tensor on the LUT's
    (CUDA) device, computed by the library's dequant export (exact lookups)."""
    if bitwidth not in (1, 2, 3, 4):
        raise ValueError(f"reference_dequant supports bitwidths 1-4, got {bitwidth}")
    lut_t = lut if torch.is_tensor(lut) else torch.from_numpy(np.asarray(lut))
    if not lut_t.is_cuda:
        raise RuntimeError("reference_dequant: the LUT must live on a CUDA device")
    blob = indices_blob if torch.is_tensor(indices_blob) else torch.from_numpy(np.asarray(indices_blob))
    blob = blob.to(lut_t.device)
    lut16 = lut_t if lut_t.dtype in (torch.float16, torch.bfloat16) else None
    packed = _lib.repack_from_idxn(blob, N, K, bitwidth)
    if lut16 is not None:
        return _lib.dequant(packed, lut16.reshape(-1, 1 << bitwidth), N, K, bitwidth, group_size).float()
    # fp32 palettes (training masters): gather with the exported codes
    codes = _lib.unpack_codes(packed, N, K, bitwidth).long()
    pal = lut_t.reshape(-1, 1 << bitwidth)
    rg = (torch.arange(N, device=pal.device) // int(group_size)).clamp_(max=pal.shape[0] - 1)
    return pal[rg].float().gather(1, codes)


class PalettizedLinear(nn.Module):
    """y = x @ W^T (+ second stream, + low-rank residual, + bias), W palettized.

    Arguments as in the reference constructor (palettized_modules.py:413-417):
    indices: idxN blob (uint8, N*K*bitwidth/8 bytes); lut: [ceil(N/gs), 2**bitwidth]
    fp16 or bf16; optional second stream (indices2, lut2, bitwidth2), residual
    factors resA [N, R] / resB [R, K], bias [N]; rotation_seed/rotation_k enable
    the Hadamard input rotation (signs drawn as the palettizer does);
    awq_scale + fold_order="rotate_then_awq" select the compensated rotation.
    """

    def __init__(self, indices, lut, bitwidth, group_size, N, K, bias=None,
                 resA=None, resB=None, indices2=None, lut2=None,
                 bitwidth2=None, reference: bool = False,
                 rotation_seed: int = None, rotation_k: int = None,
                 awq_scale=None, fold_order: str = None):
        super().__init__()
        self.N, self.K = int(N), int(K)
        self.bitwidth = int(bitwidth)
        self.bitwidth2 = self.bitwidth if bitwidth2 is None else int(bitwidth2)
        self.group_size = int(group_size)
        self.reference = bool(reference)
        self._dev_cache = {}
        self._packed = self._packed2 = None

        # --- geometry the slab / idxN layouts can express
        if self.N % 128 or self.K % 64:
            raise ValueError(f"PalettizedLinear: the code layout tiles 128 rows x 64 columns, so N%128 and "
                             f"K%64 must be 0 (N={self.N}, K={self.K})")
        for label, width in (("bitwidth", self.bitwidth), ("bitwidth2", self.bitwidth2)):
            if not 1 <= width <= 4:
                raise ValueError(f"PalettizedLinear: {label}={width}; code widths are 1, 2, 3 or 4 bits")

        # --- code streams: stream 1 always, stream 2 as a complete pair or not at all
        self.register_buffer("indices", self._checked_blob(indices, self.bitwidth, "stream 1"), persistent=False)
        self.register_buffer("lut", self._lut2d(lut, self.bitwidth), persistent=False)
        if (indices2 is None) != (lut2 is None):
            raise ValueError("PalettizedLinear: a second code stream is given by BOTH indices2 and lut2 "
                             "(one of them is missing)")
        if indices2 is None:
            self.indices2 = self.lut2 = None
        else:
            palette2 = self._lut2d(lut2, self.bitwidth2)
            if palette2.shape[0] != self.lut.shape[0]:
                raise ValueError(f"PalettizedLinear: the two streams must share one row-group grid; "
                                 f"stream 1 has {self.lut.shape[0]} palettes, stream 2 has {palette2.shape[0]}")
            self.register_buffer("indices2", self._checked_blob(indices2, self.bitwidth2, "stream 2"),
                                 persistent=False)
            self.register_buffer("lut2", palette2, persistent=False)

        # --- low-rank residual (both factors) and bias
        if resA is None or resB is None:
            self.resA = self.resB = None
        else:
            rank = resB.shape[0]
            if tuple(resA.shape) != (self.N, rank) or resB.shape[1] != self.K:
                raise ValueError(f"PalettizedLinear: residual factors must be resA [N, R] and resB [R, K]; got "
                                 f"{tuple(resA.shape)} and {tuple(resB.shape)} for N={self.N}, K={self.K}")
            self.register_buffer("resA", resA, persistent=False)
            self.register_buffer("resB", resB, persistent=False)
        if bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = nn.Parameter(bias, requires_grad=False)

        # --- input rotation: the signs are a pure function of (K, seed); an AWQ scale only makes
        #     sense on a rotated module
        self.rotation_seed = None if rotation_seed is None else int(rotation_seed)
        self.rotation_k = None if rotation_k is None else int(rotation_k)
        self.fold_order = fold_order if fold_order in ("awq_then_rotate", "rotate_then_awq") else None
        self.rot_signs = self.awq_scale = None
        rotated = self.rotation_seed is not None and self.rotation_k is not None
        if rotated and self.rotation_k != self.K:
            raise ValueError(f"PalettizedLinear: rotation_k={self.rotation_k} but the rotation acts on the "
                             f"input axis, K={self.K}")
        if awq_scale is not None and not rotated:
            raise ValueError("PalettizedLinear: awq_scale without rotation metadata (rotation_seed, rotation_k)")
        if rotated:
            self.rot_signs = _fht.rotation_signs(self.rotation_k, self.rotation_seed)
        if awq_scale is not None:
            scale = torch.as_tensor(awq_scale, dtype=torch.float32).detach().cpu()
            if scale.dim() != 1 or scale.numel() != self.K:
                raise ValueError(f"PalettizedLinear: awq_scale has shape {tuple(scale.shape)}; one value per "
                                 f"input channel (K={self.K}) is expected")
            if not bool(torch.isfinite(scale).all()) or bool((scale <= 0).any()):
                raise ValueError("PalettizedLinear: every awq_scale entry must be finite and positive")
            self.awq_scale = scale
            self.fold_order = self.fold_order or "rotate_then_awq"

    def _checked_blob(self, blob, width: int, label: str) -> torch.Tensor:
        blob = torch.as_tensor(blob)
        want = self.N * self.K * width // 8
        if blob.numel() != want:
            raise ValueError(f"PalettizedLinear: {label}: idx{width} blob numel is {blob.numel()}, "
                             f"N*K*{width}/8 = {want} bytes are needed (N={self.N}, K={self.K})")
        return blob

    @staticmethod
    def _lut2d(lut, bits):
        t = lut if torch.is_tensor(lut) else torch.from_numpy(np.asarray(lut))
        if t.dim() != 2:
            t = t.view(-1, 1 << bits)
        if t.shape[1] != (1 << bits):
            raise ValueError(f"LUT palette width {t.shape[1]} != 2**bitwidth {1 << bits}")
        return t

    # ------------------------------------------------------------------ state
    def has_residual(self) -> bool:
        return self.resA is not None and self.resB is not None

    @property
    def has_stream2(self) -> bool:
        return self.indices2 is not None and self.lut2 is not None

    def _logical_indices_numpy(self, blob=None, bits=None) -> np.ndarray:
        """(N, K) uint8 logical codes of a stream's idxN blob (host, numpy)."""
        b = int(bits) if bits is not None else self.bitwidth
        blob = self.indices if blob is None else blob
        arr = np.ascontiguousarray(blob.detach().cpu().numpy(), dtype=np.uint8).reshape(-1)
        return _idxn.unpack_idxn(arr, self.N, self.K, b)

    def _on(self, name: str, t: torch.Tensor, device) -> torch.Tensor:
        key = (name, str(device))
        v = self._dev_cache.get(key)
        if v is None:
            v = t.to(device=device, dtype=torch.float32).contiguous()
            self._dev_cache[key] = v
        return v

    def _ensure_packed(self):
        """One-time device conversion idxN blob -> slab layout (per stream)."""
        dev = self.lut.device
        if not self.lut.is_cuda:
            raise RuntimeError("PalettizedLinear: move the module to a CUDA device first "
                               "(this package has no CPU compute route)")
        if self._packed is None or self._packed.device != dev:
            self._packed = _lib.repack_from_idxn(self.indices.to(dev), self.N, self.K, self.bitwidth)
            self._packed2 = None
        if self.has_stream2 and self._packed2 is None:
            self._packed2 = _lib.repack_from_idxn(self.indices2.to(dev), self.N, self.K, self.bitwidth2)

    def drop_blob(self) -> "PalettizedLinear":
        """Free the idxN blob(s) once the slab copy exists (halves weight memory)."""
        self._ensure_packed()
        self.indices = torch.empty(0, dtype=torch.uint8, device=self.lut.device)
        if self.has_stream2:
            self.indices2 = torch.empty(0, dtype=torch.uint8, device=self.lut.device)
        return self

    @classmethod
    def from_packed(cls, packed, lut, bitwidth, group_size, N, K, **kw) -> "PalettizedLinear":
        """Build a module around codes that are already in the slab layout
        (used by the synthetic model stack, which draws random codes on the device)."""
        mod = cls.__new__(cls)
        nn.Module.__init__(mod)
        blob = torch.empty(0, dtype=torch.uint8, device=packed.device)
        mod.bitwidth, mod.bitwidth2, mod.group_size = int(bitwidth), int(bitwidth), int(group_size)
        mod.N, mod.K, mod.reference = int(N), int(K), False
        mod.register_buffer("indices", blob, persistent=False)
        mod.register_buffer("lut", cls._lut2d(lut, int(bitwidth)), persistent=False)
        mod.resA = mod.resB = mod.indices2 = mod.lut2 = None
        bias = kw.get("bias")
        mod.register_parameter("bias", None if bias is None else nn.Parameter(bias, requires_grad=False))
        mod.rotation_seed = mod.rotation_k = mod.fold_order = None
        mod.rot_signs = mod.awq_scale = None
        mod._dev_cache = {}
        mod._packed, mod._packed2 = packed, None
        if packed.numel() != N * K * bitwidth // 8:
            raise ValueError("from_packed: wrong code buffer size")
        return mod

    # ---------------------------------------------------------------- pieces
    def _segment_desc(self, out: Optional[torch.Tensor], ldo: Optional[int] = None,
                      with_bias: bool = True, res_t: Optional[torch.Tensor] = None) -> dict:
        self._ensure_packed()
        d = dict(packed=self._packed, lut=self.lut, N=self.N, group_size=self.group_size,
                 n_groups=self.lut.shape[0], bits=self.bitwidth, out=out,
                 ldo=self.N if ldo is None else ldo)
        if res_t is not None:          # fused low-rank residual: t = x @ resB^T computed by the caller
            d.update(resA=self.resA, res_t=res_t)
        if self.has_stream2:
            d.update(packed2=self._packed2, lut2=self.lut2, bits2=self.bitwidth2)
        if with_bias and self.bias is not None:
            d["bias"] = self.bias.data
        return d

    def _compute_dtype(self) -> torch.dtype:
        if self.lut.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"PalettizedLinear(kernel path): LUT dtype must be float16 or "
                             f"bfloat16, got lut ({self.lut.dtype})")
        if self.has_stream2 and self.lut2.dtype != self.lut.dtype:
            raise ValueError("PalettizedLinear(kernel path): both LUTs must share one dtype")
        if self.bias is not None and self.bias.dtype != self.lut.dtype:
            raise ValueError("PalettizedLinear(kernel path): bias dtype must equal the LUT dtype")
        return self.lut.dtype

    def _rotate_input(self, x: torch.Tensor) -> torch.Tensor:
        signs = self._on("signs", self.rot_signs, x.device)
        if self.awq_scale is not None and self.fold_order == "rotate_then_awq":
            return _fht.fht_apply_awq(x, signs, self._on("awq", self.awq_scale, x.device))
        return _fht.fht_apply(x, signs)

    def _fusable_residual(self, M: int, dtype: torch.dtype) -> bool:
        """Rank a multiple of 8, factors in the compute dtype and 16-byte aligned: the residual
        rides the projection launch. At decode (M <= 16) a projection launch computes
        t = x @ resB^T in fp32 and the GEMV epilogue adds t @ resA^T; at prefill t is rounded to
        the compute dtype (as the reference route does) and enters the tensor-core GEMM's
        accumulator as extra k-blocks — one-stream launches with at most two palettes per
        128-row tile, and the two-stream launch pair."""
        if M > GEMV_MAX_M and not self._prefill_residual_served():
            return False
        return (self.has_residual() and M > 0 and self.resA.shape[1] <= 1024
                and self.resA.shape[1] % 8 == 0 and self.resA.dtype == dtype
                and self.resB.dtype == dtype and self.resA.is_contiguous()
                and self.resB.is_contiguous() and self.resA.data_ptr() % 16 == 0
                and self.resB.data_ptr() % 16 == 0)

    def _prefill_residual_served(self) -> bool:
        if self.group_size < 64 or self.K < 128:
            return False
        if not self.has_stream2:
            return True
        return not (self.bitwidth == 4 and self.bitwidth2 == 4)   # the 4 + 4 pair is one one-tile launch

    def _rotation_fuses(self, M: int, dtype=None) -> bool:
        """The input rotation can run inside the decode launch: 4-bit single stream, at most 8
        rows, no low-rank residual (its projection needs the rotated row in memory), K made of
        at most 8 power-of-two segments."""
        return (self.rot_signs is not None and not self.reference and 0 < M <= 8 and self.bitwidth == 4
                and (dtype is None or dtype == self.lut.dtype)      # else the rotation rounds in x's dtype
                and not self.has_stream2 and not self.has_residual() and self.group_size >= 32
                and bin(self.K).count("1") <= 8
                and os.environ.get("FLUTE_NO_FHT_FUSE", "").strip() not in ("1", "true", "True"))

    def _rows_kernel_shape(self, M: int, dtype) -> bool:
        """What the row-range decode kernel serves (and with it every input transform)."""
        return (not self.reference and 0 < M <= 8 and self.bitwidth == 4 and not self.has_stream2
                and self.group_size >= 32 and dtype == self.lut.dtype
                and self.lut.dtype in (torch.float16, torch.bfloat16))

    def _fold(self, device):
        """(rot_signs, awq_scale) of this module's input fold on `device`, (None, None) if unrotated."""
        if self.rot_signs is None:
            return None, None
        awq = None
        if self.awq_scale is not None and self.fold_order == "rotate_then_awq":
            awq = self._on("awq", self.awq_scale, device)
        return self._on("signs", self.rot_signs, device), awq

    def forward_gated(self, g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        """self(silu(g) * u) for 2-D g, u of one shape: at decode the product (and this module's
        rotation) runs in the prologue of the projection launch; otherwise one elementwise pass
        over g and the ordinary forward."""
        M = g.shape[0]
        strided = (g.stride(1) == 1 and u.stride(1) == 1 and g.stride(0) == u.stride(0) and g.stride(0) % 8 == 0)
        if (g.dtype == u.dtype and strided and self._rows_kernel_shape(M, g.dtype)
                and not self.has_residual() and g.data_ptr() % 16 == 0 and u.data_ptr() % 16 == 0
                and (self.rot_signs is None or self._rotation_fuses(M, g.dtype))):
            out = torch.empty(M, self.N, dtype=g.dtype, device=g.device)
            signs, awq = self._fold(g.device)
            inp = _lib.make_input(x_mul=u, rot_signs=signs, awq_scale=awq)
            _lib.gemv_input(g, _lib.make_segments([self._segment_desc(out)]), 1, inp, flags=_flags())
            return out
        g = g.contiguous()
        _lib.silu_mul(g, u)
        return self(g)

    def _input_transform(self, device):
        signs = self._on("signs", self.rot_signs, device)
        awq = None
        if self.awq_scale is not None and self.fold_order == "rotate_then_awq":
            awq = self._on("awq", self.awq_scale, device)
        return _lib.make_input(rot_signs=signs, awq_scale=awq)

    def _kernel_matmul(self, x2: torch.Tensor, fuse_residual: bool = False,
                       fuse_rotation: bool = False) -> torch.Tensor:
        """x2 [M, K] in the compute dtype -> [M, N] (streams + bias, and the low-rank
        residual when fuse_residual; fuse_rotation: x2 is the UNROTATED row and the launch
        rotates it)."""
        M = x2.shape[0]
        out = torch.empty(M, self.N, dtype=x2.dtype, device=x2.device)
        if M == 0:
            return out
        res_t = None
        if fuse_residual:
            project = _lib.residual_project if M <= GEMV_MAX_M else _lib.residual_project_rows
            res_t = project(x2, self.resB, flags=_flags())
        segs = _lib.make_segments([self._segment_desc(out, res_t=res_t)])
        if fuse_rotation:
            _lib.gemv_input(x2, segs, 1, self._input_transform(x2.device), flags=_flags())
        elif M <= GEMV_MAX_M:
            _lib.gemv_multi(x2, segs, 1, flags=_flags())
        elif (self.bitwidth == 4 and (not self.has_stream2 or self.bitwidth2 == 4)) or \
                (not self.has_stream2 and self.group_size >= 64 and self.K >= 128):
            # tensor-core GEMM: any width for one code stream with at most two palettes per
            # tile; 4-bit codes for the two-stream and group-size-32 forms
            _lib.gemm(x2, segs, flags=_flags())
        elif self.has_stream2 and self.group_size >= 64 and self.K >= 128:
            # two streams of different widths: one tensor-core launch per stream, fp32 sums
            # carried from the first to the second, one rounding
            _lib.gemm_two_stream(x2, segs, flags=_flags())
        else:
            # what the tensor-core GEMM does not serve: decode kernel, 16 rows at a time
            for r0 in range(0, M, GEMV_MAX_M):
                rows = slice(r0, min(M, r0 + GEMV_MAX_M))
                _lib.gemv_multi(x2[rows], _lib.make_segments([self._segment_desc(out[rows])]), 1,
                                flags=_flags())
        return out

    def _reference_matmul(self, x2: torch.Tensor) -> torch.Tensor:
        """The reference route's arithmetic on the GPU: exact dequant, fp32
        matmul per stream, ordered fp32 add, one rounding; bias added after."""
        self._ensure_packed()
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            xf = x2.float()
            w1 = self._dequant_stream(self._packed, self.lut, self.bitwidth)
            y = xf @ w1.t()
            if self.has_stream2:
                y = y + xf @ self._dequant_stream(self._packed2, self.lut2, self.bitwidth2).t()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        return y.to(x2.dtype)

    def _dequant_stream(self, packed, lut, bits) -> torch.Tensor:
        if lut.dtype in (torch.float16, torch.bfloat16):
            return _lib.dequant(packed, lut, self.N, self.K, bits, self.group_size).float()
        codes = _lib.unpack_codes(packed, self.N, self.K, bits).long()
        rg = (torch.arange(self.N, device=lut.device) // self.group_size).clamp_(max=lut.shape[0] - 1)
        return lut[rg].float().gather(1, codes)

    def _quantized_weight(self) -> torch.Tensor:
        """Effective dequantised weight W1 (+ W2), fp32 [N, K], in the module's
        (fold-space) basis."""
        self._ensure_packed()
        w = self._dequant_stream(self._packed, self.lut, self.bitwidth)
        if self.has_stream2:
            w = w + self._dequant_stream(self._packed2, self.lut2, self.bitwidth2)
        return w

    # --------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("PalettizedLinear.forward: x must be a CUDA tensor")
        shape = x.shape
        if x.shape[-1] != self.K:
            raise ValueError(f"PalettizedLinear: input feature dim {x.shape[-1]} != K {self.K}")
        if self.K == 0 or self.N == 0 or x.numel() == 0:
            # degenerate shapes of the reference's kernels: K == 0 gives zeros (+ bias),
            # N == 0 or no rows give an empty result (kernel_streaming.cu:2363-2368)
            out = torch.zeros(*shape[:-1], self.N, dtype=x.dtype, device=x.device)
            return out + self.bias.to(x.dtype) if self.bias is not None and self.N else out
        x2 = x.reshape(-1, self.K)
        fuse_rotation = self._rotation_fuses(x2.shape[0], x2.dtype)
        if self.rot_signs is not None and not fuse_rotation:
            x2 = self._rotate_input(x2)
        if self.reference:
            out = self._reference_matmul(x2)
            bias_done = False
        else:
            cd = self._compute_dtype()
            xc = x2 if x2.dtype == cd else x2.to(cd)
            if xc.stride(-1) != 1 or xc.stride(0) % 8 or xc.data_ptr() % 16:
                xc = xc.contiguous().clone() if xc.data_ptr() % 16 else xc.contiguous()
            residual_done = self._fusable_residual(xc.shape[0], xc.dtype)
            out = self._kernel_matmul(xc, fuse_residual=residual_done, fuse_rotation=fuse_rotation).to(x.dtype)
            bias_done = True
        if self.has_residual() and not (not self.reference and residual_done):
            xr = x2.to(self.resA.dtype)
            out = out + ((xr @ self.resB.t()) @ self.resA.t()).to(out.dtype)
        if self.bias is not None and not bias_done:
            out = out + self.bias
        return out.reshape(*shape[:-1], self.N)


def _per_segment_folds(mods, M: int) -> bool:
    """The projections carry different folds, yet one launch can serve them: each block of the
    row-range kernel rotates the shared rows with the fold of the segment it works on (the
    reference's merged kernels carry a fold per segment the same way,
    src/flute_extended/src/kernel_gemv_multi.cu:101-334)."""
    dt = mods[0].lut.dtype
    for m in mods:
        if not m._rows_kernel_shape(M, dt):
            return False
        if m.rot_signs is not None and not m._rotation_fuses(M, dt):
            return False
    return True


def _mergeable(mods, x: torch.Tensor, per_segment: bool = False) -> bool:
    """Decode-merge decision: M <= 16, same K, one dtype, unrotated or one shared rotation (or,
    with per_segment, folds the launch can apply per segment), and every low-rank residual of
    a kind the GEMV epilogue serves."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.shape[0] > GEMV_MAX_M or x2.shape[0] == 0 or not x.is_cuda:
        return False
    m0 = mods[0]
    if not all(isinstance(m, PalettizedLinear) for m in mods):
        return False
    one_fold = all(_same_rotation(m0, m) for m in mods)
    if not one_fold and not (per_segment and all(m.K == m0.K and m.lut.dtype == m0.lut.dtype for m in mods)
                             and _per_segment_folds(mods, x2.shape[0])):
        return False
    for m in mods:
        if not isinstance(m, PalettizedLinear) or m.reference or m.K != m0.K:
            return False
        if m.lut.dtype != m0.lut.dtype:
            return False
        if m.lut.dtype not in (torch.float16, torch.bfloat16):
            return False
        if m.has_residual() and not m._fusable_residual(x2.shape[0], m.lut.dtype):
            return False
    return True


def _prefill_mergeable(mods, x: torch.Tensor) -> bool:
    """Prefill-merge decision (M > 16): projections that share x run as ONE tensor-core launch
    when they have one code stream each, one code width, one group size >= 64, one dtype, only
    low-rank residuals the launch can carry, and are unrotated or share one rotation."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.shape[0] <= GEMV_MAX_M or not x.is_cuda or len(mods) > _lib.GEMM_MULTI_MAX:
        return False
    if os.environ.get("FLUTE_NO_MERGE", "").strip() in ("1", "true", "True"):
        return False
    m0 = mods[0]
    for m in mods:
        if not isinstance(m, PalettizedLinear) or m.reference or m.K != m0.K or m.K < 128:
            return False
        if m.lut.dtype != m0.lut.dtype or m.lut.dtype not in (torch.float16, torch.bfloat16):
            return False
        if m.has_stream2 or not _same_rotation(m0, m):
            return False
        if m.has_residual() and not m._fusable_residual(x2.shape[0], m.lut.dtype):
            return False
        if m.bitwidth != m0.bitwidth or m.group_size != m0.group_size or m.group_size < 64:
            return False
        if m.bias is not None and m.bias.dtype != m.lut.dtype:
            return False
    return True


def _prefill_merged(mods, x: torch.Tensor, outs) -> None:
    """One merged prefill launch of `mods` over x into the 2-D buffers `outs` (each [M, >= N]
    with its own row stride)."""
    m0 = mods[0]
    x2 = x.reshape(-1, x.shape[-1])
    if m0.rot_signs is not None:
        x2 = m0._rotate_input(x2)
    x2 = x2.to(m0.lut.dtype).contiguous()
    # the residual projections' t blocks lie side by side in one matrix
    widths = [_lib.residual_block_cols(m.resB.shape[0]) if m.has_residual() else 0 for m in mods]
    t_all = torch.empty(x2.shape[0], sum(widths), dtype=x2.dtype, device=x2.device) if any(widths) else None
    descs, col = [], 0
    for m, o, w in zip(mods, outs, widths):
        res_t = None
        if w:
            res_t = _lib.residual_project_rows(x2, m.resB, flags=_flags(), out=t_all[:, col:col + w])
            col += w
        descs.append(m._segment_desc(o, ldo=o.stride(0), res_t=res_t))
    _lib.gemm_multi(x2, _lib.make_segments(descs), len(descs), flags=_flags())


def _same_rotation(a: "PalettizedLinear", b: "PalettizedLinear") -> bool:
    """Both unrotated, or both rotated by the same fold (seed, length, order, AWQ scale): a
    merged launch rotates the shared input row once. Different folds merge only where the
    launch itself can rotate per segment (_per_segment_folds)."""
    if a.rot_signs is None or b.rot_signs is None:
        return a.rot_signs is None and b.rot_signs is None
    if (a.rotation_seed, a.rotation_k, a.fold_order) != (b.rotation_seed, b.rotation_k, b.fold_order):
        return False
    if a.awq_scale is None or b.awq_scale is None:
        return a.awq_scale is None and b.awq_scale is None
    return a is b or torch.equal(a.awq_scale, b.awq_scale)


def _stacked_residual(owner: nn.Module, mods, x2: torch.Tensor):
    """One projection launch for all residuals of a merged launch: the rB factors are
    stacked once (cached on the owner), t = x2 @ stack^T, and each module gets its slice."""
    with_res = [m for m in mods if m.has_residual()]
    if not with_res:
        return {}
    key = tuple(m.resB.data_ptr() for m in with_res)
    cache = owner.__dict__.get("_resB_stack")
    if cache is None or cache[0] != key:
        cache = (key, torch.cat([m.resB for m in with_res], dim=0).contiguous())
        owner.__dict__["_resB_stack"] = cache
    t = _lib.residual_project(x2, cache[1], flags=_flags())
    out, off = {}, 0
    for m in with_res:
        r = m.resB.shape[0]
        out[id(m)] = t[:, off:off + r]
        off += r
    return out


def _merged_decode(owner: nn.Module, mods, x: torch.Tensor, epilogue: int = None) -> torch.Tensor:
    """One decode launch for projections that share x (their outputs side by side in one
    [M, sum N] buffer; under the SiLU*mul epilogue only the gate's). One shared fold runs as a
    transform launch in front — or inside the launch where the row-range kernel serves it;
    different folds always run inside the launch, one per segment."""
    epi = _lib.EPI_NONE if epilogue is None else epilogue
    cd = mods[0].lut.dtype
    x2 = x.reshape(-1, x.shape[-1])
    M = x2.shape[0]
    m0 = mods[0]
    one_fold = all(_same_rotation(m0, m) for m in mods)
    inp = None
    if not one_fold:
        inp = _lib.make_input(seg_folds=[m._fold(x.device) for m in mods])
    elif m0.rot_signs is not None:
        if all(m._rows_kernel_shape(M, cd) and m._rotation_fuses(M, x2.dtype) for m in mods):
            inp = m0._input_transform(x.device)
        else:
            x2 = m0._rotate_input(x2)
    x2 = x2.to(cd).contiguous()
    silu = epi == _lib.EPI_SILU_MUL
    total = mods[0].N if silu else sum(m.N for m in mods)
    out = torch.empty(M, total, dtype=cd, device=x.device)
    res = _stacked_residual(owner, mods, x2) if inp is None or not one_fold else {}
    descs, off = [], 0
    for i, m in enumerate(mods):
        dst = None if (silu and i % 2) else out[:, off:]
        descs.append(m._segment_desc(dst, ldo=total, res_t=res.get(id(m))))
        if dst is not None:
            off += m.N
    segs = _lib.make_segments(descs)
    if inp is not None:
        _lib.gemv_input(x2, segs, len(descs), inp, epilogue=epi, flags=_flags())
    else:
        _lib.gemv_multi(x2, segs, len(descs), epilogue=epi, flags=_flags())
    return out


class SplitQKV(nn.Module):
    """q/k/v projections sharing one input: one merged decode launch when
    M <= 16, else the three modules (reference palettized_modules.py:1390-1466)."""

    def __init__(self, q_proj, k_proj, v_proj):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = q_proj, k_proj, v_proj

    def forward(self, x):
        mods = (self.q_proj, self.k_proj, self.v_proj)
        if _prefill_mergeable(mods, x):      # M > 16: one tensor-core launch for the three
            total = sum(m.N for m in mods)
            M = x.numel() // x.shape[-1]
            out = torch.empty(M, total, dtype=mods[0].lut.dtype, device=x.device)
            offs = [0, mods[0].N, mods[0].N + mods[1].N]
            _prefill_merged(mods, x, [out[:, o:] for o in offs])
            return out.to(x.dtype).reshape(*x.shape[:-1], total)
        if os.environ.get("FLUTE_NO_MERGE", "").strip() in ("1", "true", "True") \
                or not _mergeable(mods, x, per_segment=True):
            return torch.cat([m(x) for m in mods], dim=-1)
        out = _merged_decode(self, mods, x)
        return out.to(x.dtype).reshape(*x.shape[:-1], out.shape[1])


class FusedPalettizedMLP(nn.Module):
    """down(act(gate(x)) * up(x)); at M <= 16 with a SiLU activation the gate and
    up projections and the SiLU*mul run as ONE launch (fp32 silu on the fp32 sums,
    one rounding) (reference palettized_modules.py:1643-1723)."""

    def __init__(self, gate_proj, up_proj, down_proj, act_fn):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.act_fn = act_fn

    def _is_silu(self) -> bool:
        return isinstance(self.act_fn, nn.SiLU) or self.act_fn in (torch.nn.functional.silu,)

    def fused_gate_up(self, x2: torch.Tensor) -> torch.Tensor:
        """silu(gate(x2)) * up(x2) for rows already in the projections' basis, one launch."""
        g, u = self.gate_proj, self.up_proj
        out = torch.empty(x2.shape[0], g.N, dtype=x2.dtype, device=x2.device)
        res = _stacked_residual(self, (g, u), x2)
        descs = [g._segment_desc(out, res_t=res.get(id(g))), u._segment_desc(None, res_t=res.get(id(u)))]
        epi = _lib.EPI_SILU_MUL
        if x2.shape[0] <= GEMV_MAX_M:
            _lib.gemv_multi(x2, _lib.make_segments(descs), 2, epilogue=epi, flags=_flags())
        else:
            raise RuntimeError("fused gate/up is a decode (M <= 16) route")
        return out

    def forward(self, x):
        mods = (self.gate_proj, self.up_proj)
        merge = (self._is_silu() and mods[0].N == mods[1].N
                 and os.environ.get("FLUTE_NO_MERGE", "").strip() not in ("1", "true", "True"))
        fusable = merge and _mergeable(mods, x)
        if not fusable and merge and _mergeable(mods, x, per_segment=True):
            # gate and up carry different folds: one launch rotates the shared rows per segment
            # and leaves g | u side by side; SiLU*mul then runs in the prologue of the down launch
            gu = _merged_decode(self, mods, x)
            n = mods[0].N
            y = self.down_proj.forward_gated(gu[:, :n], gu[:, n:])
            return y.to(x.dtype).reshape(*x.shape[:-1], self.down_proj.N)
        if not fusable:
            if self._is_silu() and mods[0].N == mods[1].N and _prefill_mergeable(mods, x):
                # prefill: gate and up as one tensor-core launch, one SiLU*mul pass, down
                M = x.numel() // x.shape[-1]
                g = torch.empty(M, mods[0].N, dtype=mods[0].lut.dtype, device=x.device)
                u = torch.empty_like(g)
                _prefill_merged(mods, x, [g, u])
                _lib.silu_mul(g, u)
                y = self.down_proj(g.to(x.dtype))
                return y.reshape(*x.shape[:-1], self.down_proj.N)
            g, u = self.gate_proj(x), self.up_proj(x)
            if (self._is_silu() and g.is_cuda and g.dtype in (torch.float16, torch.bfloat16)
                    and g.dtype == u.dtype and g.shape[-1] % 8 == 0 and g.is_contiguous()
                    and u.is_contiguous() and not self.gate_proj.reference):
                # prefill: one SiLU*mul pass over the two projections' outputs
                _lib.silu_mul(g.view(-1, g.shape[-1]), u.view(-1, u.shape[-1]))
                return self.down_proj(g)
            return self.down_proj(self.act_fn(g) * u)
        y = _merged_decode(self, mods, x, epilogue=_lib.EPI_SILU_MUL).to(x.dtype)
        return self.down_proj(y).reshape(*x.shape[:-1], self.down_proj.N)


class PalettizedEmbedding(nn.Module):
    """Embedding over a palettized [N, K] table: forward(ids) gathers rows.

    Drop-in for the reference's PalettizedEmbedding
    (src/scripts/palettized_modules.py:1979-2335): same constructor signature,
    attribute names and dtype ladder —
        w   = lut1[id // gs][idx1[id]] (+ lut2[id // gs][idx2[id]], one add in the palette
              dtype, stream 1 first)
        out = (w.float() + resA[id].float() @ resB.float())  [-> adjoint Hadamard transform
              when the table is a tied, rotated head]  -> palette dtype, ONE rounding.
    The reference gathers through torch indexing over an unpacked [N, K] uint8 copy of the
    codes; here one CUDA launch (b200lut_embed_gather) reads the rows out of the packed slab
    layout, so a table tied to an lm_head (`tied_to`) shares that module's codes and nothing
    is unpacked. There is no CPU route, and no trainable-palette mode.

    Ids outside [0, N): CPU ids raise ValueError like the reference; for CUDA ids the
    reference aborts the context with a device-side assertion, this module writes a row of
    zeros and raises the library's device status (`_lib.lib().b200lut_device_status()`),
    without a host synchronisation.
    """

    def __init__(self, indices, lut, bitwidth, group_size, N, K, indices2=None, lut2=None,
                 bitwidth2=None, resA=None, resB=None, num_embeddings=None, embedding_dim=None,
                 rotation_seed: int = None, rotation_k: int = None):
        super().__init__()
        self.bitwidth = int(bitwidth)
        if self.bitwidth not in (1, 2, 3, 4):
            raise ValueError(f"PalettizedEmbedding: bitwidth {self.bitwidth} not in 1..4 — the idxN "
                             f"artifact family is the contract")
        self.bitwidth2 = int(bitwidth2) if bitwidth2 is not None else self.bitwidth
        if self.bitwidth2 not in (1, 2, 3, 4):
            raise ValueError(f"PalettizedEmbedding: bitwidth2 {self.bitwidth2} not in 1..4 — the "
                             f"idxN artifact family is the contract")
        self.group_size = int(group_size)
        self.N, self.K = int(N), int(K)
        if num_embeddings is not None and int(num_embeddings) != self.N:
            raise ValueError(f"PalettizedEmbedding: num_embeddings {num_embeddings} != N {self.N}; "
                             f"the two spellings must agree")
        if embedding_dim is not None and int(embedding_dim) != self.K:
            raise ValueError(f"PalettizedEmbedding: embedding_dim {embedding_dim} != K {self.K}; "
                             f"the two spellings must agree")
        if self.N % 128 != 0 or self.K % 64 != 0:
            raise ValueError(f"idxN layout requires N%128==0 and K%64==0, got N={self.N}, K={self.K}")
        indices = torch.as_tensor(indices)
        expected = (self.N * self.K * self.bitwidth) // 8
        if indices.numel() != expected:
            raise ValueError(f"idx{self.bitwidth} blob numel {indices.numel()} != "
                             f"N*K*{self.bitwidth}/8 {expected} (N={self.N}, K={self.K})")
        self.register_buffer("indices", indices, persistent=False)
        self.register_buffer("lut", PalettizedLinear._lut2d(lut, self.bitwidth), persistent=False)
        if resA is not None and resB is not None:
            if resA.shape != (self.N, resB.shape[0]) or resB.shape[1] != self.K:
                raise ValueError(f"residual factors shape mismatch: A {tuple(resA.shape)}, "
                                 f"B {tuple(resB.shape)} for N={self.N}, K={self.K}")
            self.register_buffer("resA", resA, persistent=False)
            self.register_buffer("resB", resB, persistent=False)
        else:
            self.resA = self.resB = None
        if indices2 is None and lut2 is None:
            self.indices2 = self.lut2 = None
        elif indices2 is None or lut2 is None:
            raise ValueError("PalettizedEmbedding: a second stream needs BOTH indices2 and lut2; "
                             "refusing a half-constructed two-stream module")
        else:
            indices2 = torch.as_tensor(indices2)
            expected2 = (self.N * self.K * self.bitwidth2) // 8
            if indices2.numel() != expected2:
                raise ValueError(f"idx{self.bitwidth2} stream-2 blob numel {indices2.numel()} != "
                                 f"N*K*{self.bitwidth2}/8 {expected2} (N={self.N}, K={self.K})")
            lut2_t = PalettizedLinear._lut2d(lut2, self.bitwidth2)
            if lut2_t.shape[0] != self.lut.shape[0]:
                raise ValueError(f"stream-2 LUT groups {lut2_t.shape[0]} != stream-1 "
                                 f"{self.lut.shape[0]}; both streams must share the group grid")
            self.register_buffer("indices2", indices2, persistent=False)
            self.register_buffer("lut2", lut2_t, persistent=False)
        self.rotation_seed = int(rotation_seed) if rotation_seed is not None else None
        self.rotation_k = int(rotation_k) if rotation_k is not None else None
        self.rot_signs = None
        self._signs_cache = {}
        if self.rotation_seed is not None and self.rotation_k is not None:
            if self.rotation_k != self.K:
                raise ValueError(f"PalettizedEmbedding: rotation_k {self.rotation_k} != the embedding "
                                 f"dim K {self.K} — corrupt rotation record on a tied artifact set")
            self.rot_signs = _fht.rotation_signs(self.rotation_k, self.rotation_seed)
        self._packed = None
        self._packed2 = None
        self._tied = []          # [PalettizedLinear] whose slab copies serve this table
        self._bad_ids = None     # device flag: a forward met a CUDA id outside [0, N)

    @classmethod
    def tied_to(cls, lm: PalettizedLinear) -> "PalettizedEmbedding":
        """The embedding consumer of a tied head: the SAME buffers as `lm` (blobs, palettes,
        residual factors) and the same slab copy of the codes; inherits the head's rotation
        record, so gathered rows are un-rotated (reference load_tied_pair, :2792-2872)."""
        emb = cls(lm.indices, lm.lut, lm.bitwidth, lm.group_size, lm.N, lm.K,
                  indices2=lm.indices2, lut2=lm.lut2,
                  bitwidth2=lm.bitwidth2 if lm.has_stream2 else None, resA=lm.resA, resB=lm.resB,
                  rotation_seed=lm.rotation_seed, rotation_k=lm.rotation_k) \
            if lm.indices.numel() else None
        if emb is None:           # the head already dropped its blob: build around its slab copy
            emb = cls.__new__(cls)
            nn.Module.__init__(emb)
            emb.bitwidth, emb.bitwidth2, emb.group_size = lm.bitwidth, lm.bitwidth2, lm.group_size
            emb.N, emb.K = lm.N, lm.K
            for name in ("indices", "lut", "resA", "resB", "indices2", "lut2"):
                v = getattr(lm, name)
                if v is None:
                    setattr(emb, name, None)
                else:
                    emb.register_buffer(name, v, persistent=False)
            emb.rotation_seed, emb.rotation_k = lm.rotation_seed, lm.rotation_k
            emb.rot_signs, emb._signs_cache = lm.rot_signs, {}
            emb._packed = emb._packed2 = None
            emb._bad_ids = None
        emb._tied = [lm]
        return emb

    # the nn.Embedding spellings
    @property
    def num_embeddings(self) -> int:
        return self.N

    @property
    def embedding_dim(self) -> int:
        return self.K

    def has_residual(self) -> bool:
        return self.resA is not None and self.resB is not None

    @property
    def has_stream2(self) -> bool:
        return self.indices2 is not None and self.lut2 is not None

    def _logical_indices_numpy(self, blob=None, bits=None) -> np.ndarray:
        """(N, K) uint8 logical codes of a stream's idxN blob (host, numpy)."""
        b = int(bits) if bits is not None else self.bitwidth
        blob = self.indices if blob is None else blob
        arr = np.ascontiguousarray(blob.detach().cpu().numpy(), dtype=np.uint8).reshape(-1)
        return _idxn.unpack_idxn(arr, self.N, self.K, b)

    def _signs_on(self, device) -> torch.Tensor:
        key = str(device)
        v = self._signs_cache.get(key)
        if v is None:
            v = self.rot_signs.to(device=device, dtype=torch.float32).contiguous()
            self._signs_cache[key] = v
        return v

    def _table(self) -> dict:
        dev = self.lut.device
        if not self.lut.is_cuda:
            raise RuntimeError("PalettizedEmbedding: move the module to a CUDA device first "
                               "(this package has no CPU compute route)")
        if self.lut.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"PalettizedEmbedding: LUT dtype must be float16 or bfloat16, got "
                             f"{self.lut.dtype}")
        if self._tied and self._tied[0].lut.device == dev:
            lm = self._tied[0]
            lm._ensure_packed()
            p1, p2 = lm._packed, lm._packed2
        else:
            if self._packed is None or self._packed.device != dev:
                self._packed = _lib.repack_from_idxn(self.indices.to(dev), self.N, self.K, self.bitwidth)
                self._packed2 = None
            if self.has_stream2 and self._packed2 is None:
                self._packed2 = _lib.repack_from_idxn(self.indices2.to(dev), self.N, self.K,
                                                      self.bitwidth2)
            p1, p2 = self._packed, self._packed2
        d = dict(packed=p1, lut=self.lut, bits=self.bitwidth, N=self.N, group_size=self.group_size,
                 n_groups=self.lut.shape[0])
        if self.has_stream2:
            d.update(packed2=p2, lut2=self.lut2.to(self.lut.dtype), bits2=self.bitwidth2)
        if self.has_residual():
            if (self.resA.dtype != self.lut.dtype or self.resB.dtype != self.lut.dtype) \
                    and not self.__dict__.get("_warned_residual_dtype"):
                # the reference widens the factors to fp32 in the dtype they are stored in
                # (src/scripts/palettized_modules.py:2320); the gather kernel reads them in
                # the palette dtype, so wider factors lose their extra bits here
                import warnings
                warnings.warn(f"PalettizedEmbedding: residual factors in {self.resA.dtype} / {self.resB.dtype} are "
                              f"rounded to the palette dtype {self.lut.dtype} for the gather kernel")
                self.__dict__["_warned_residual_dtype"] = True
            d.update(resA=self.resA.to(self.lut.dtype).contiguous(),
                     resB=self.resB.to(self.lut.dtype).contiguous())
        return d

    def forward(self, ids):
        if not torch.is_tensor(ids):
            ids = torch.as_tensor(ids)
        if ids.dtype not in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
            raise ValueError(f"PalettizedEmbedding.forward: ids must be an integer tensor, got dtype "
                             f"{ids.dtype}")
        if not ids.is_cuda and ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= self.N):
            raise ValueError(f"PalettizedEmbedding.forward: ids out of range [0, {self.N}) (min "
                             f"{int(ids.min())}, max {int(ids.max())}); refusing a silent wrap")
        table = self._table()
        flat = ids.to(device=self.lut.device, dtype=torch.int64).reshape(-1).contiguous()
        if ids.is_cuda and flat.numel():
            # Device-resident ids cannot be refused here without a host sync (the reference
            # asserts on the device, which would lose the context). The kernel writes zeros for
            # such an id; the module remembers that it happened, without a sync, and
            # check_ids() raises at a moment the host chooses.
            bad = ((flat < 0) | (flat >= self.N)).any()
            self._bad_ids = bad if self._bad_ids is None else (self._bad_ids | bad)
        dtype = self.lut.dtype
        if self.rot_signs is None:
            out = _lib.embed_gather(flat, table, self.K, dtype)
        else:
            w = _lib.embed_gather(flat, table, self.K, dtype, out_fp32=True)
            if flat.numel():
                w = _lib.fht(w, self._signs_on(w.device), _lib.FHT_ADJOINT, out=w)
            out = _lib.round_rows(w, dtype)
        return out.view(*ids.shape, self.K)


    def check_ids(self) -> None:
        """Raise if any forward since the last check met a CUDA id outside [0, N) (those rows
        were gathered as zeros). Synchronises once; clears the record and the library's device
        status word (0x6000) that the gather kernel raised."""
        bad, self._bad_ids = self._bad_ids, None
        if bad is not None and bool(bad.item()):
            _lib.lib().b200lut_device_status()
            raise ValueError(f"PalettizedEmbedding: ids out of range [0, {self.N}) were gathered as "
                             f"zero rows since the last check")


class KGroupedPalettizedLinear(nn.Module):
    """Linear layer whose palettes are grouped along the INPUT axis: one 2**bitwidth-entry
    palette per (block of 128 input columns, output row),
        W[n, k] = lut_k[k // 128][n][idx[n, k]],   y = x @ W^T (+ bias), fp32 sums, one rounding.
    The reference has no module of this form (its groups run along the output rows); in its
    terms this is K/128 PalettizedLinear(group_size=1, K=128) modules summed in fp32
    (src/scripts/palettized_modules.py:125-162). indices: the idxN blob of the [N, K] codes;
    lut_k: [K // 128, N, 2**bitwidth] float16 / bfloat16. Up to 16 rows run the decode kernel
    (b200lut_gemv_kgrouped), more the tensor-core GEMM (b200lut_gemm_kgrouped)."""

    GROUP_K = 128

    def __init__(self, indices, lut_k, bitwidth, N, K, bias=None):
        super().__init__()
        self.bitwidth, self.N, self.K = int(bitwidth), int(N), int(K)
        if self.bitwidth not in (1, 2, 3, 4):
            raise ValueError(f"KGroupedPalettizedLinear: bitwidth must be 1-4, got {self.bitwidth}")
        if self.N % 128 != 0 or self.K % 128 != 0:
            raise ValueError(f"KGroupedPalettizedLinear needs N%128==0 and K%128==0, got N={self.N}, "
                             f"K={self.K}")
        indices = torch.as_tensor(indices)
        expected = (self.N * self.K * self.bitwidth) // 8
        if indices.numel() != expected:
            raise ValueError(f"idx{self.bitwidth} blob numel {indices.numel()} != N*K*{self.bitwidth}/8 "
                             f"{expected} (N={self.N}, K={self.K})")
        lut_k = torch.as_tensor(lut_k)
        want = (self.K // self.GROUP_K, self.N, 1 << self.bitwidth)
        if tuple(lut_k.shape) != want:
            raise ValueError(f"lut_k shape {tuple(lut_k.shape)} != (K/128, N, 2**bitwidth) = {want}")
        self.register_buffer("indices", indices, persistent=False)
        self.register_buffer("lut_k", lut_k.contiguous(), persistent=False)
        self.register_parameter("bias", None if bias is None else nn.Parameter(bias, requires_grad=False))
        self._packed = None

    def _ensure_packed(self):
        dev = self.lut_k.device
        if not self.lut_k.is_cuda:
            raise RuntimeError("KGroupedPalettizedLinear: move the module to a CUDA device first "
                               "(this package has no CPU compute route)")
        if self.lut_k.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"KGroupedPalettizedLinear: palette dtype must be float16 or bfloat16, "
                             f"got {self.lut_k.dtype}")
        if self._packed is None or self._packed.device != dev:
            self._packed = _lib.repack_from_idxn(self.indices.to(dev), self.N, self.K, self.bitwidth)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.K:
            raise ValueError(f"KGroupedPalettizedLinear: input feature dim {x.shape[-1]} != K {self.K}")
        if not x.is_cuda:
            raise RuntimeError("KGroupedPalettizedLinear: x must be a CUDA tensor")
        self._ensure_packed()
        cd = self.lut_k.dtype
        x2 = x.reshape(-1, self.K).to(cd).contiguous()
        M = x2.shape[0]
        out = torch.empty(M, self.N, dtype=cd, device=x.device)
        bias = None if self.bias is None else self.bias.data.to(cd)
        if M == 0:
            return out.to(x.dtype).reshape(*x.shape[:-1], self.N)
        if M <= GEMV_MAX_M:
            _lib.gemv_kgrouped(x2, self._packed, self.lut_k, self.N, self.bitwidth, bias=bias, out=out)
        else:
            _lib.gemm_kgrouped(x2, self._packed, self.lut_k, self.N, self.bitwidth, bias=bias, out=out,
                               flags=_flags())
        return out.to(x.dtype).reshape(*x.shape[:-1], self.N)
