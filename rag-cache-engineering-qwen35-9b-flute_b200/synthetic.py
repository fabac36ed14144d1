"""Seeded synthetic tensors with the shapes and value distributions of the
Qwen3.5-9B palettized projections (stand-ins for real artifacts).

codes: uniform integers in [0, 2**bits); palette: 0.02 * randn sorted ascending
along the palette axis, cast to the operand dtype; activations: randn.
Seed convention: BASE_SEED + configuration index.
"""
from __future__ import annotations

import numpy as np
import torch

from . import idxN

BASE_SEED = 20261125


def make_codes(N: int, K: int, bits: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, 1 << bits, size=(N, K), dtype=np.uint8)


def make_blob(N: int, K: int, bits: int, seed: int):
    """(codes [N, K] uint8, idxN blob uint8 tensor) on the host."""
    codes = make_codes(N, K, bits, seed)
    return codes, torch.from_numpy(idxN.pack_idxn(codes, bits))


def make_lut(n_groups: int, bits: int, dtype: torch.dtype, seed: int, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (std * torch.randn(n_groups, 1 << bits, generator=g)).sort(dim=1).values.to(dtype)


def make_x(M: int, K: int, dtype: torch.dtype, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).to(dtype)


def random_blob_on_device(N: int, K: int, bits: int, seed: int, device) -> torch.Tensor:
    """A uniformly random idxN blob drawn on the device. Every byte pattern is a
    valid blob and uniform bytes are uniform codes, so this equals packing
    uniform random codes without the host round trip (used at 9B scale)."""
    g = torch.Generator(device=device).manual_seed(seed)
    n = N * K * bits // 8
    return torch.randint(0, 256, (n,), dtype=torch.uint8, device=device, generator=g)
