"""Pin the CPU oracle to outputs of the reference's own code (tests/golden/).

Every comparison is bit-exact: integer work by equality, floating work by
torch.equal on the result tensors (the oracle restates the same torch ops in the
same order; summation order is fixed by running single-threaded).
"""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

from oracle import lut_linear_oracle as orc

IDXN_SHAPES = ((128, 64), (256, 128), (384, 192), (1024, 512))


def _sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


@pytest.fixture(autouse=True)
def _single_thread():
    n = torch.get_num_threads()
    torch.set_num_threads(1)
    yield
    torch.set_num_threads(n)


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
def test_pack_unpack_matches_reference_blobs(golden, bits):
    # same generator stream as the reference self-test (seed 0, widths ascending)
    rng = np.random.default_rng(0)
    for b in (1, 2, 3, 4):
        for (N, K) in IDXN_SHAPES:
            idx = rng.integers(0, 1 << b, size=(N, K), dtype=np.uint8)
            if b != bits:
                continue
            tag = f"idxn_b{b}_{N}x{K}"
            blob = orc.pack_idxn(idx, b)
            if golden.has(tag + "_blob"):
                assert np.array_equal(idx, golden.np(tag + "_idx"))
                assert np.array_equal(blob, golden.np(tag + "_blob"))
            else:
                assert np.array_equal(_sha(idx), golden.np(tag + "_idx_sha"))
                assert np.array_equal(_sha(blob), golden.np(tag + "_blob_sha"))
            assert np.array_equal(orc.unpack_idxn(blob, N, K, b), idx)


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
def test_scalar_unpack_agrees(golden, bits):
    tag = f"idxn_b{bits}_128x64"
    got = orc.unpack_idxn_scalar(golden.np(tag + "_blob"), 128, 64, bits)
    assert np.array_equal(got, golden.np(tag + "_idx"))


def test_unpack_refuses_wrong_width_and_shape():
    idx = np.zeros((128, 64), dtype=np.uint8)
    blob = orc.pack_idxn(idx, 3)
    with pytest.raises(ValueError):
        orc.unpack_idxn(blob, 128, 64, 4)
    with pytest.raises(ValueError):
        orc.pack_idxn(np.zeros((100, 64), dtype=np.uint8), 4)
    with pytest.raises(ValueError):
        orc.pack_idxn(np.zeros((128, 60), dtype=np.uint8), 4)
    with pytest.raises(ValueError):
        orc.pack_idxn(np.full((128, 64), 9, dtype=np.uint8), 3)


@pytest.mark.parametrize("case", range(4))
def test_dequant_bit_exact(golden, case):
    N, K, gs, b, groups = (int(v) for v in golden.np(f"deq{case}_meta"))
    lut = golden.t(f"deq{case}_lut")
    assert lut.shape[0] == groups
    W = orc.dequant(golden.np(f"deq{case}_blob"), lut, N, K, gs, b)
    assert W.dtype == torch.float32
    assert torch.equal(W, golden.t(f"deq{case}_W"))


@pytest.mark.parametrize("case", range(7))
def test_forward_bit_exact(golden, case):
    tag = f"fwd{case}"
    N, K, gs, b, M, b2, rank, has_bias, rot_seed, awq, x3d = (int(v) for v in golden.np(tag + "_meta"))
    lut = golden.t(tag + "_lut")
    w1 = orc.dequant(golden.np(tag + "_blob"), lut, N, K, gs, b)
    w2 = None
    if b2 > 0:
        w2 = orc.dequant(golden.np(tag + "_blob2"), golden.t(tag + "_lut2"), N, K, gs, b2)
    signs = None
    if rot_seed >= 0:
        signs = orc.rotation_signs(K, rot_seed)
        assert torch.equal(signs, golden.t(tag + "_signs"))
    y = orc.linear_forward(golden.t(tag + "_x"), w1, w2,
                           resA=golden.opt(tag + "_resA"), resB=golden.opt(tag + "_resB"),
                           bias=golden.opt(tag + "_bias"), rot_signs=signs,
                           awq_scale=golden.opt(tag + "_awq") if awq else None)
    want = golden.t(tag + "_y")
    assert y.dtype == want.dtype and y.shape == want.shape
    assert torch.equal(y, want)


@pytest.mark.parametrize("K,seed", ((64, 0), (1024, 7), (1024, 42), (4096, 0), (12288, 3)))
def test_rotation_signs_pinned(golden, K, seed):
    s = orc.rotation_signs(K, seed)
    assert s.dtype == torch.float32 and set(s.unique().tolist()) <= {-1.0, 1.0}
    assert np.array_equal(s.to(torch.int8).numpy(), golden.np(f"signs_K{K}_s{seed}"))


def test_segments():
    assert orc.fht_segments(4096) == [(0, 4096)]
    assert orc.fht_segments(12288) == [(0, 8192), (8192, 4096)]
    assert orc.fht_segments(6144) == [(0, 4096), (4096, 2048)]
    assert orc.fht_segments(192) == [(0, 128), (128, 64)]


@pytest.mark.parametrize("case", range(4))
def test_fht_bit_exact(golden, case):
    M, K, seed = (int(v) for v in golden.np(f"fht{case}_meta"))
    x = golden.t(f"fht{case}_x")
    s = orc.rotation_signs(K, seed)
    assert torch.equal(orc.fht_forward(x, s), golden.t(f"fht{case}_fwd"))
    assert torch.equal(orc.fht_adjoint(x, s), golden.t(f"fht{case}_adj"))
    assert torch.equal(orc.fht_forward_awq(x, s, golden.t(f"fht{case}_scale")),
                       golden.t(f"fht{case}_awq"))


def test_fht_block128(golden):
    assert torch.equal(orc.fht_block(golden.t("fhtblk_x"), 128), golden.t("fhtblk_y"))


@pytest.mark.parametrize("seed", (7, 42))
def test_fht_matches_explicit_matrix(seed):
    # the reference's own gate (src/rag/tests/test_turboquant.py:88-103):
    # |x@T - fht(x)| < 1e-4 and the adjoint round trip < 1e-5 at D = 1024
    D = 1024
    s = orc.rotation_signs(D, seed)
    x = torch.randn(8, D, generator=torch.Generator().manual_seed(seed))
    T = orc.rotation_matrix(s)
    y = orc.fht_forward(x, s)
    assert (y - x @ T).abs().max().item() < 1e-4
    assert (orc.fht_adjoint(y, s) - x).abs().max().item() < 1e-5


def test_kgrouped_composition():
    rng = np.random.default_rng(5)
    N, K = 128, 256
    idx = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    lut_k = (0.02 * torch.randn(K // 128, N, 16, generator=torch.Generator().manual_seed(5))).bfloat16()
    W = orc.dequant_kgrouped(idx, lut_k, 128)
    n, k = 77, 200
    assert W[n, k].item() == float(lut_k[k // 128, n, idx[n, k]])
    assert W.shape == (N, K)


def test_fused_silu_mul_close_to_unfused():
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(1, 256, generator=g), torch.randn(1, 256, generator=g)
    fused = orc.silu_mul_fused(a, b, torch.bfloat16)
    unfused = torch.nn.functional.silu(a.bfloat16()) * b.bfloat16()
    assert orc.max_rel_err(fused, unfused.float()) < 2e-2


EMBED_CASES = ("e1", "e2", "e3", "e4", "e5", "e6", "e7")


@pytest.mark.parametrize("name", EMBED_CASES)
def test_embedding_forward_matches_reference_module(golden_embedding, name):
    g = golden_embedding
    N, K, gs, bits, bits2, rank, rot = (int(v) for v in g.np(name + "_meta"))
    signs = orc.rotation_signs(K, rot) if rot >= 0 else None
    got = orc.embedding_forward(
        g.t(name + "_ids"), g.np(name + "_codes"), g.t(name + "_lut"), gs,
        idx2=g.np(name + "_codes2") if bits2 else None, lut2=g.opt(name + "_lut2"),
        resA=g.opt(name + "_resA"), resB=g.opt(name + "_resB"), rot_signs=signs)
    want = g.t(name + "_out")
    assert got.dtype == want.dtype and got.shape == want.shape
    assert torch.equal(got, want)


def test_embedding_forward_refuses_ids_outside_the_table(golden_embedding):
    g = golden_embedding
    with pytest.raises(ValueError):
        orc.embedding_forward(torch.tensor([256]), g.np("e1_codes"), g.t("e1_lut"), 64)
    with pytest.raises(ValueError):
        orc.embedding_forward(torch.tensor([-1]), g.np("e1_codes"), g.t("e1_lut"), 64)
