"""Hadamard boundary-fold rotation of the activations, served by the CUDA library.

Mirrors the interface of the reference's src/flute_extended/fht.py
(rotation_signs :105, segments :118, hadamard_matrix :137,
build_rotation_matrix :151, fht_apply :528, fht_apply_awq :583, fht_adjoint
:655, fht_apply_ :698) with one compute backend: b200lut_fht on CUDA tensors.
There is no torch or CPU twin in this package; non-CUDA inputs are refused.

T is block-diagonal over the descending power-of-two segments of K
(4096 -> [4096]; 12288 -> [8192, 4096]); per segment T = H diag(signs) / sqrt(b).
fht_block() is the additional sign-free fixed-block form (e.g. 128-point blocks).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from . import _lib

__all__ = ["rotation_signs", "segments", "hadamard_matrix", "build_rotation_matrix",
           "fht_apply", "fht_apply_awq", "fht_adjoint", "fht_apply_", "fht_block",
           "kernel_available"]


def rotation_signs(K: int, seed: int) -> torch.Tensor:
    """(K,) float32 vector of +-1: CPU generator seeded seed + 4242,
    randint(0, 2) * 2 - 1 (the palettizer's draw; reference fht.py:105-115)."""
    g = torch.Generator().manual_seed(int(seed) + 4242)
    return torch.randint(0, 2, (int(K),), generator=g).float().mul(2).sub(1)


def segments(K: int) -> List[Tuple[int, int]]:
    """Descending power-of-two decomposition [(offset, size), ...]."""
    K = int(K)
    if K < 1:
        raise ValueError("segments: K must be >= 1")
    out, off = [], 0
    while off < K:
        b = 1 << ((K - off).bit_length() - 1)
        out.append((off, b))
        off += b
    return out


def hadamard_matrix(K: int) -> torch.Tensor:
    """Sylvester H_K (+-1 entries); test/diagnostic materialisation only."""
    K = int(K)
    if K < 1 or K & (K - 1):
        raise ValueError("hadamard_matrix needs a power-of-two size")
    H = torch.ones(1, 1)
    while H.shape[0] < K:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return H


def build_rotation_matrix(K: int, seed: int, device=None) -> torch.Tensor:
    """Explicit (K, K) fp32 T for (K, seed) — ground truth for differential tests."""
    s = rotation_signs(K, seed)
    T = torch.zeros(K, K)
    for off, b in segments(K):
        T[off:off + b, off:off + b] = hadamard_matrix(b) * s[off:off + b].view(1, b) / math.sqrt(b)
    return T.to(device) if device is not None else T


def kernel_available(x: Optional[torch.Tensor] = None) -> bool:
    """True when the CUDA library is loadable (and x, if given, is on CUDA)."""
    try:
        _lib.lib()
    except (RuntimeError, OSError):
        return False
    return True if x is None else bool(x.is_cuda)


def _check(x: torch.Tensor, signs: torch.Tensor, backend: str) -> Tuple[int, int]:
    if backend not in ("auto", "kernel"):
        raise ValueError(f"fht: backend {backend!r} is not served; this package has one backend, "
                         "the CUDA kernel ('auto' or 'kernel')")
    if signs.dim() != 1 or signs.numel() != x.shape[-1]:
        raise ValueError(f"fht: signs must be a (K,) vector matching x's last dim "
                         f"(got signs {tuple(signs.shape)}, x {tuple(x.shape)})")
    if not torch.is_floating_point(x):
        raise TypeError(f"fht: x must be floating point, got {x.dtype}")
    if not x.is_cuda:
        raise RuntimeError("fht: x must be a CUDA tensor (no CPU route in this package)")
    K = int(x.shape[-1])
    return x.numel() // K, K


def _vec(v: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return v.detach().to(device=x.device, dtype=torch.float32).contiguous()


def _run(x: torch.Tensor, signs, mode: int, scale=None, block: int = 0, out=None) -> torch.Tensor:
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    y = _lib.fht(x2, signs, mode=mode, scale=scale, block=block, out=out)
    return y.reshape(x.shape)


class _FhtFn(torch.autograd.Function):
    """y = x @ T (adjoint=False) or x @ T^T (adjoint=True); the backward of one
    is the other (reference fht.py:485-525)."""

    @staticmethod
    def forward(ctx, x, signs, adjoint):
        ctx.save_for_backward(signs)
        ctx.adjoint = adjoint
        return _run(x, signs, _lib.FHT_ADJOINT if adjoint else _lib.FHT_FORWARD)

    @staticmethod
    def backward(ctx, grad):
        (signs,) = ctx.saved_tensors
        g = _run(grad.contiguous(), signs, _lib.FHT_FORWARD if ctx.adjoint else _lib.FHT_ADJOINT)
        return g, None, None


def fht_apply(x: torch.Tensor, signs: torch.Tensor, backend: str = "auto") -> torch.Tensor:
    """out = x @ T. x: (..., K) fp16/bf16/fp32 on CUDA; fp32 butterfly; out in x.dtype."""
    _check(x, signs, backend)
    s = _vec(signs, x)
    if x.requires_grad:
        return _FhtFn.apply(x, s, False)
    return _run(x, s, _lib.FHT_FORWARD)


def fht_adjoint(v: torch.Tensor, signs: torch.Tensor, backend: str = "auto") -> torch.Tensor:
    """out = v @ T^T (signs on the input side)."""
    _check(v, signs, backend)
    s = _vec(signs, v)
    if v.requires_grad:
        return _FhtFn.apply(v, s, True)
    return _run(v, s, _lib.FHT_ADJOINT)


def fht_apply_awq(x: torch.Tensor, signs: torch.Tensor, s: torch.Tensor,
                  backend: str = "auto") -> torch.Tensor:
    """out = ((x * s) @ T) / s in one kernel: fp32 multiply on load, true fp32
    division on store (reference fht.py:583-652)."""
    _check(x, signs, backend)
    if s.dim() != 1 or s.numel() != x.shape[-1]:
        raise ValueError(f"fht_awq: s must be a (K,) vector matching x's last dim "
                         f"(got s {tuple(s.shape)}, x last dim {x.shape[-1]})")
    if not torch.is_floating_point(s):
        raise TypeError(f"fht_awq: s must be floating point, got {s.dtype}")
    if x.requires_grad:
        raise RuntimeError("fht_apply_awq: autograd is not served on the compensated form")
    return _run(x, _vec(signs, x), _lib.FHT_AWQ, scale=_vec(s, x))


def fht_apply_(x: torch.Tensor, signs: torch.Tensor, backend: str = "auto") -> torch.Tensor:
    """In-place x <- x @ T (no-grad only)."""
    if x.requires_grad:
        raise RuntimeError("fht_apply_: in-place FHT on a tensor that requires grad — use "
                           "fht_apply (out-of-place) for autograd correctness")
    _check(x, signs, backend)
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or x2.data_ptr() != x.data_ptr():
        x.copy_(fht_apply(x, signs))
        return x
    _lib.fht(x2, _vec(signs, x), mode=_lib.FHT_FORWARD, out=x2)
    return x


def fht_block(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Normalised, sign-free Hadamard transform of every `block`-wide slice of
    the last dim (the prefill variant: a 128-point block rotation)."""
    if not x.is_cuda:
        raise RuntimeError("fht_block: x must be a CUDA tensor")
    return _run(x, None, _lib.FHT_FORWARD, block=int(block))
