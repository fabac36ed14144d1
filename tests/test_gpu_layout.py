"""GPU parity, integer/byte work (bit-exact): idxN blob -> slab layout and back,
code export, and the dequantised-weight export against the oracle and the
reference-made golden tiles."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import pkg
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
@pytest.mark.parametrize("shape", ((128, 64), (256, 192), (384, 512), (1024, 1024)))
def test_repack_round_trips(bits, shape):
    N, K = shape
    codes = np.random.default_rng(bits * 100 + N).integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
    blob = torch.from_numpy(orc.pack_idxn(codes, bits)).cuda()
    packed = L.repack_from_idxn(blob, N, K, bits)
    assert packed.numel() == N * K * bits // 8
    assert np.array_equal(L.unpack_codes(packed, N, K, bits).cpu().numpy(), codes)
    assert torch.equal(L.repack_to_idxn(packed, N, K, bits), blob)


def test_repack_is_a_permutation_of_bit_strings():
    # all-ones codes stay all ones; a single set code lands in exactly `bits` bits
    N, K, bits = 128, 64, 3
    codes = np.zeros((N, K), np.uint8)
    codes[77, 13] = 7
    packed = L.repack_from_idxn(torch.from_numpy(orc.pack_idxn(codes, bits)).cuda(), N, K, bits)
    assert int(np.unpackbits(packed.cpu().numpy()).sum()) == 3


@pytest.mark.parametrize("case", range(4))
def test_dequant_matches_reference_golden(golden, case):
    N, K, gs, b, groups = (int(v) for v in golden.np(f"deq{case}_meta"))
    lut = golden.t(f"deq{case}_lut").cuda()
    packed = L.repack_from_idxn(torch.from_numpy(golden.np(f"deq{case}_blob")).cuda(), N, K, b)
    W = L.dequant(packed, lut, N, K, b, gs)
    assert W.dtype == lut.dtype
    assert torch.equal(W.float().cpu(), golden.t(f"deq{case}_W"))


@pytest.mark.parametrize("bits,gs,dtype", ((4, 128, torch.bfloat16), (3, 64, torch.float16),
                                           (4, 32, torch.float16), (2, 256, torch.bfloat16)))
def test_dequant_bit_exact_large(bits, gs, dtype):
    N, K = 1024, 2048
    rng = np.random.default_rng(7)
    codes = rng.integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
    lut = (0.02 * torch.randn(N // gs, 1 << bits, generator=torch.Generator().manual_seed(7))).to(dtype)
    want = orc.dequant_indices(codes, lut, gs, bits)
    packed = L.repack_from_idxn(torch.from_numpy(orc.pack_idxn(codes, bits)).cuda(), N, K, bits)
    got = L.dequant(packed, lut.cuda(), N, K, bits, gs)
    assert torch.equal(got.float().cpu(), want)
    ref = pkg.reference_dequant(torch.from_numpy(orc.pack_idxn(codes, bits)), lut.cuda(), N, K, gs, bits)
    assert ref.dtype == torch.float32 and torch.equal(ref.cpu(), want)


def test_full_size_projection_round_trip_property():
    # 12288 x 4096 at 4 bits: random blob drawn on the device; blob -> slab -> blob
    N, K, bits = 12288, 4096, 4
    blob = pkg.synthetic.random_blob_on_device(N, K, bits, 11, "cuda")
    packed = L.repack_from_idxn(blob, N, K, bits)
    assert torch.equal(L.repack_to_idxn(packed, N, K, bits), blob)
    # code histogram is preserved by the permutation
    codes = L.unpack_codes(packed, N, K, bits)
    lo, hi = blob & 15, blob >> 4
    want = torch.bincount(lo.long(), minlength=16) + torch.bincount(hi.long(), minlength=16)
    assert torch.equal(torch.bincount(codes.flatten().long(), minlength=16), want)
