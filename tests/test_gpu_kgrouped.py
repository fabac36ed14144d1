"""GPU parity of the K-grouped palette variant (one palette per 128 input columns and output
row) against the oracle composition of reference calls (oracle.dequant_kgrouped: per K block a
reference dequantisation with group_size = 1, concatenated along K; then the reference
forward's fp32 matmul and one rounding).

Dequantised weights BIT-EXACT (one-hot activations); outputs max rel err <= 1e-2."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, pkg, rel_err
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib


def _case(N, K, bits, dtype, seed, bias=False):
    rng = np.random.default_rng(seed)
    g = torch.Generator().manual_seed(seed)
    codes = rng.integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
    lut_k = (0.02 * torch.randn(K // 128, N, 1 << bits, generator=g)).sort(dim=-1).values.to(dtype)
    b = (0.1 * torch.randn(N, generator=g)).to(dtype) if bias else None
    mod = pkg.KGroupedPalettizedLinear(torch.from_numpy(orc.pack_idxn(codes, bits)), lut_k, bits, N, K,
                                       bias=b).cuda()
    return codes, lut_k, b, mod


@pytest.mark.parametrize("N,K,bits,dtype,M,bias", (
    (4096, 4096, 4, torch.bfloat16, 1, False),     # the single-projection configuration
    (256, 128, 4, torch.float16, 3, True),         # one column group
    (384, 1024, 3, torch.bfloat16, 8, False),
    (128, 512, 2, torch.float16, 16, True),
    (512, 256, 1, torch.bfloat16, 5, False),
    (1024, 2048, 4, torch.bfloat16, 40, True),     # more than 16 rows: served 16 at a time
))
def test_outputs_match_the_oracle_composition(N, K, bits, dtype, M, bias):
    codes, lut_k, b, mod = _case(N, K, bits, dtype, N + K + M, bias)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(dtype)
    got = mod(x.cuda())
    want = orc.linear_forward(x, orc.dequant_kgrouped(codes, lut_k, 128), bias=b)
    assert got.shape == (M, N) and got.dtype == dtype
    assert rel_err(got, want) <= TOL
    assert torch.equal(mod(x.cuda()), got)           # deterministic, tickets reset themselves


@pytest.mark.parametrize("bits,dtype", ((4, torch.bfloat16), (3, torch.float16), (2, torch.bfloat16),
                                        (1, torch.float16)))
def test_dequantised_weights_are_bit_exact(bits, dtype):
    N, K = 256, 256
    codes, lut_k, _, mod = _case(N, K, bits, dtype, 10 + bits)
    W = mod(torch.eye(K, dtype=dtype, device="cuda")).cpu().t()      # [N, K]
    assert torch.equal(W.float(), orc.dequant_kgrouped(codes, lut_k, 128).float())


def test_every_split_gives_the_same_sums_within_rounding():
    N, K, M = 256, 2048, 4
    codes, lut_k, _, mod = _case(N, K, 4, torch.bfloat16, 99)
    mod._ensure_packed()
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    want = orc.linear_forward(x.cpu(), orc.dequant_kgrouped(codes, lut_k, 128))
    for split in (1, 2, 5, 16):
        got = L.gemv_kgrouped(x, mod._packed, mod.lut_k, N, 4, split=split)
        assert rel_err(got, want) <= TOL, split
    assert L.lib().b200lut_gemv_kgrouped_split(4096, 4096) >= 1


def test_refusals():
    codes, lut_k, _, mod = _case(128, 128, 4, torch.bfloat16, 1)
    mod._ensure_packed()
    x = torch.zeros(17, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="M <= 16"):
        L.gemv_kgrouped(x, mod._packed, mod.lut_k, 128, 4)
    with pytest.raises(RuntimeError, match="exceeds"):
        L.gemv_kgrouped(x[:1], mod._packed, mod.lut_k, 128, 4, split=2)
    with pytest.raises(ValueError, match="lut_k shape"):
        pkg.KGroupedPalettizedLinear(mod.indices.cpu(), lut_k[:, :64], 4, 128, 128)
    with pytest.raises(ValueError, match="K%128"):
        pkg.KGroupedPalettizedLinear(torch.zeros(128 * 64 // 2, dtype=torch.uint8), lut_k, 4, 128, 64)
