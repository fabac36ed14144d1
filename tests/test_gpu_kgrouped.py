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
    (1024, 2048, 4, torch.bfloat16, 40, True),     # more than 16 rows: the tensor-core form
    (4096, 4096, 4, torch.bfloat16, 300, True),    # 64 tiles: cut in two along K over the idle SMs
    (512, 1024, 3, torch.float16, 128, False),
    (256, 256, 2, torch.bfloat16, 257, True),      # a second token tile of one row
    (128, 128, 1, torch.float16, 17, False),       # one tile, two k-blocks, one palette block
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


@pytest.mark.parametrize("bits,dtype", ((4, torch.bfloat16), (3, torch.float16), (2, torch.bfloat16),
                                        (1, torch.float16)))
def test_weights_through_the_tensor_core_form_are_bit_exact(bits, dtype):
    N, K = 384, 256
    codes, lut_k, _, mod = _case(N, K, bits, dtype, 20 + bits)
    mod._ensure_packed()
    W = L.gemm_kgrouped(torch.eye(K, dtype=dtype, device="cuda"), mod._packed, mod.lut_k, N, bits).cpu().t()
    assert torch.equal(W.float(), orc.dequant_kgrouped(codes, lut_k, 128).float())
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0


def test_tensor_core_form_at_prefill_width_sampled():
    # M = 2048, K = 4096, N = 4096: every token, 256 sampled weight rows; both schedules agree
    N, K, M, dt = 4096, 4096, 2048, torch.bfloat16
    codes, lut_k, _, mod = _case(N, K, 4, dt, 4242)
    mod._ensure_packed()
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).to(dt).cuda()
    got = L.gemm_kgrouped(x, mod._packed, mod.lut_k, N, 4)
    whole = L.gemm_kgrouped(x, mod._packed, mod.lut_k, N, 4, split=False)
    rows = torch.cat([torch.arange(t * 128, t * 128 + 64) for t in (0, 11, 20, 31)])
    w = orc.dequant_kgrouped(codes[rows.numpy()], lut_k[:, rows], 128)
    want = orc.linear_forward(x.cpu(), w)
    assert rel_err(got[:, rows.cuda()], want) <= TOL
    assert rel_err(got, whole) <= 4e-3
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0


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


def test_the_shared_scratch_survives_a_change_of_shape():
    # the wrapper keeps one scratch per stream: its tickets sit where a smaller shape left
    # partial sums, so a larger shape after a smaller one must still fold correctly
    dt = torch.bfloat16
    for N, K, M, bits in ((256, 2048, 2, 3), (1536, 2048, 16, 3), (512, 4096, 9, 4), (2048, 1024, 16, 4)):
        codes, lut_k, _, mod = _case(N, K, bits, dt, N + K)
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(N)).to(dt)
        want = orc.linear_forward(x, orc.dequant_kgrouped(codes, lut_k, 128))
        for _ in range(2):
            assert rel_err(mod(x.cuda()), want) <= TOL, (N, K, M, bits)


@pytest.mark.parametrize("N,K,M,dtype", ((4096, 4096, 1, torch.bfloat16), (12288, 4096, 3, torch.float16),
                                         (4096, 12288, 8, torch.bfloat16), (160 * 32, 256, 5, torch.bfloat16),
                                         (128, 128, 2, torch.float16)))
def test_row_range_form_of_the_decode_kernel(N, K, M, dtype):
    """4-bit codes at M <= 8 run the row-range form (split = 0); an explicit split keeps the
    workspace-folded kernel: both match the oracle composition and each other within rounding."""
    codes, lut_k, b, mod = _case(N, K, 4, dtype, N + K + M, bias=True)
    mod._ensure_packed()
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(dtype)
    rows = np.arange(0, N, max(1, N // 256))
    want = orc.linear_forward(x, orc.dequant_kgrouped(codes[rows], lut_k[:, rows], 128), bias=b[rows])
    got = L.gemv_kgrouped(x.cuda(), mod._packed, mod.lut_k, N, 4, bias=mod.bias.data)
    assert rel_err(got[:, rows], want) <= TOL
    again = L.gemv_kgrouped(x.cuda(), mod._packed, mod.lut_k, N, 4, bias=mod.bias.data)
    assert torch.equal(got, again)
    other = L.gemv_kgrouped(x.cuda(), mod._packed, mod.lut_k, N, 4, bias=mod.bias.data, split=2 if K >= 256 else 1)
    assert rel_err(got, other) <= 4e-3
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0
