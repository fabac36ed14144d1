"""The `flute_extended`-compatible surface: names, gates and argument checks on the CPU; one
call per compute entry on the GPU, each against the CPU oracle.

The reference's wrappers live in src/flute_extended/flute_extended/__init__.py:138-1109; its own
GPU gate for them is src/flute_extended/test_flute.py (random A ~ N(0,1), uniform codes,
LUT ~ N(0,1), M=256, K=512, N=256, gs=32)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, Case, pkg, rel_err
from oracle import lut_linear_oracle as orc

fx = pkg.flute_extended

REFERENCE_NAMES = (
    "qgemm_per_group_lut", "qgemm_dense", "qgemm_dual_stream", "qgemm_gemv_stream", "qgemm_gemv_splitk_stream",
    "qgemm_gemv_multi", "qgemm_gemv_mlp", "dual_stream_available", "dual_stream_supported",
    "gemv_stream_available", "gemv_stream_supported", "gemv_fht_stream_available", "gemv_fht_stream_supported",
    "gemv_splitk_available", "gemv_splitk_fht_available", "gemv_splitk_supported", "gemv_splitk_fht_supported",
    "gemv_multi_available", "gemv_multi_supported", "gemv_mlp_available", "gemv_mlp_supported",
    "gemv_split_hint", "DUAL_STREAM_PAIRS", "DUAL_STREAM_GROUP_SIZES", "DUAL_STREAM_MAX_M",
    "GEMV_STREAM_PAIRS", "GEMV_STREAM_GROUP_SIZES", "GEMV_SPLITK_PAIRS", "GEMV_SPLITK_GROUP_SIZES",
    "GEMV_SPLITK_MAX_RESIDUAL_RANK", "pack_idxn", "unpack_idxn")


def test_surface_has_every_name_of_the_reference_package():
    for name in REFERENCE_NAMES:
        assert hasattr(fx, name), name
    assert fx.idxN.pack_idxn is fx.pack_idxn
    # the reference's tables are subsets of what this library serves
    for pair in ((1, 4), (4, 1), (2, 3), (2, 4), (3, 3), (3, 0), (4, 0)):
        assert pair in fx.DUAL_STREAM_PAIRS and pair in fx.GEMV_STREAM_PAIRS and pair in fx.GEMV_SPLITK_PAIRS
    assert {64, 128, 256, 512} <= fx.DUAL_STREAM_GROUP_SIZES
    assert {64, 128, 256, 512, 1024, 2048} <= fx.GEMV_STREAM_GROUP_SIZES
    assert fx.DUAL_STREAM_MAX_M == 16 and fx.GEMV_SPLITK_MAX_RESIDUAL_RANK >= 256


def test_gates_mirror_the_library_contract():
    assert fx.dual_stream_available() and fx.gemv_multi_available() and fx.gemv_mlp_available()
    assert fx.dual_stream_supported(4, 0, 128, 4096, 4096)
    assert fx.dual_stream_supported(3, 3, 64, 1024, 4096)
    assert not fx.dual_stream_supported(4, 0, 128, 4000, 4096)       # N % 128
    assert not fx.dual_stream_supported(4, 0, 128, 4096, 4000)       # K % 64
    assert not fx.dual_stream_supported(5, 0, 128, 4096, 4096)       # width
    assert not fx.dual_stream_supported(4, 0, 48, 4096, 4096)        # group size
    assert fx.gemv_stream_supported(4, 1, 128, 4096, 4096, 1)
    assert not fx.gemv_stream_supported(4, 1, 128, 4096, 4096, 17)
    assert fx.gemv_splitk_supported(4, 4, 32, 1024, 12288, 1, residual_rank=32)
    assert not fx.gemv_splitk_supported(4, 4, 32, 1024, 12288, 1, residual_rank=12)
    assert fx.gemv_multi_supported(4096, 64, [(4, 0, 128), (3, 3, 64), (4, 1, 128)])
    assert not fx.gemv_multi_supported(4096, 64, [(4, 0, 128)] * 9)
    assert fx.gemv_mlp_supported(4096, 12288, [(4, 0, 128), (4, 0, 128)])
    assert not fx.gemv_mlp_supported(4096, 12288, [(4, 0, 128)])


def test_argument_checks_without_a_gpu():
    A = torch.zeros(1, 64, dtype=torch.float16)
    blob, lut = torch.zeros(128 * 64 // 2, dtype=torch.uint8), torch.zeros(1, 16, dtype=torch.float16)
    with pytest.raises(ValueError, match="indices_layout"):
        fx.qgemm_per_group_lut(A, blob, lut, 4, 128, indices_layout="idx5")
    with pytest.raises(ValueError, match="bitwidth"):
        fx.qgemm_per_group_lut(A, blob, lut, 3, 128, indices_layout="idx4")
    with pytest.raises(ValueError, match="CUDA"):
        fx.qgemm_per_group_lut(A, blob, lut, 4, 128)
    with pytest.raises(ValueError, match="cutlass_dense"):
        fx.qgemm_dense(A, torch.zeros(8, 64, dtype=torch.float16), backend="auto")
    with pytest.raises(ValueError, match="seg_table"):
        fx.qgemm_gemv_multi(A, torch.zeros(3, 14, dtype=torch.int64))
    # the dense baseline is a plain matmul
    W = torch.randn(8, 64)
    assert torch.allclose(fx.qgemm_dense(torch.ones(2, 64), W), torch.ones(2, 64) @ W.t())


# ---------------------------------------------------------------------------------------- GPU
gpu = pytest.mark.gpu


@gpu
def test_per_group_lut_shape_of_the_reference_gate():
    # src/flute_extended/test_flute.py: M=256, K=512, N=256, gs=32, LUT ~ N(0,1)
    for bits in (1, 2, 3, 4):
        case = Case(256, 512, 32, bits, torch.float16, seed=43 + bits, lut_std=1.0)
        x = case.x(256).cuda()
        y = fx.qgemm_per_group_lut(x, case.blob.cuda(), case.lut.cuda(), bits, 32, indices_layout=f"idx{bits}")
        assert y.shape == (256, 256) and y.dtype == torch.float16
        assert rel_err(y, case.oracle(x.cpu())) <= TOL
        y1 = fx.qgemm_per_group_lut(x[:1], case.blob.cuda(), case.lut.cuda(), bits, 32, indices_layout=f"idx{bits}")
        assert rel_err(y1, case.oracle(x[:1].cpu())) <= TOL


@gpu
@pytest.mark.parametrize("entry", ("qgemm_dual_stream", "qgemm_gemv_stream", "qgemm_gemv_splitk_stream"))
def test_fused_decode_entries(entry):
    case = Case(512, 1024, 128, 4, torch.bfloat16, seed=5, bits2=2, bias=True, residual=16)
    M = 5 if entry == "qgemm_dual_stream" else 1
    x = case.x(M).cuda()
    kw = dict(indices2=case.kw["indices2"].cuda(), lut2=case.kw["lut2"].cuda(), bitwidth2=2,
              resB=case.resB.cuda(), resA=case.resA.cuda(), bias=case.bias.cuda())
    y = getattr(fx, entry)(x, case.blob.cuda(), case.lut.cuda(), 4, 128, **kw)
    assert rel_err(y, case.oracle(x.cpu())) <= TOL
    # absent operands as empty tensors, the reference's convention
    plain = Case(512, 1024, 128, 4, torch.bfloat16, seed=6)
    e8, e16 = torch.empty(0, dtype=torch.uint8, device="cuda"), torch.empty(0, dtype=torch.bfloat16, device="cuda")
    y = getattr(fx, entry)(x, plain.blob.cuda(), plain.lut.cuda(), 4, 128, e8, e16, 0, e16, e16, e16)
    assert rel_err(y, plain.oracle(x.cpu())) <= TOL


@gpu
def test_gemv_entry_with_rotation_and_awq():
    case = Case(256, 4096, 128, 4, torch.float16, seed=8, rotation_seed=3, awq=True)
    x = case.x(1).cuda()
    y = fx.qgemm_gemv_splitk_stream(x, case.blob.cuda(), case.lut.cuda(), 4, 128,
                                    rot_signs=case.signs.cuda(), awq_scale=case.awq.cuda())
    assert rel_err(y, case.oracle(x.cpu())) <= TOL


def _table(rows):
    t = torch.zeros(len(rows), 15, dtype=torch.int64)
    cols = ("q1", "lut1", "q2", "lut2", "resB", "resA", "bias", "C", "N", "R", "b1", "b2", "gs", "signs", "s")
    for i, r in enumerate(rows):
        for j, c in enumerate(cols):
            t[i, j] = int(r.get(c, 0))
    return t


@gpu
def test_multi_and_mlp_tables():
    K, dt = 1024, torch.float16
    cases = [Case(256, K, 128, 4, dt, seed=21, bias=True), Case(128, K, 64, 3, dt, seed=22, bits2=3),
             Case(512, K, 128, 4, dt, seed=23, residual=8)]
    x = cases[0].x(1).cuda()
    out = torch.full((1, sum(c.N for c in cases)), float("nan"), dtype=dt, device="cuda")
    keep, rows, off = [], [], 0
    for c in cases:
        d = dict(q1=c.blob.cuda(), lut1=c.lut.cuda())
        if c.w2 is not None:
            d.update(q2=c.kw["indices2"].cuda(), lut2=c.kw["lut2"].cuda())
        if c.bias is not None:
            d["bias"] = c.bias.cuda()
        if c.resA is not None:
            d.update(resA=c.resA.cuda(), resB=c.resB.cuda())
        keep.append(d)
        r = {k: v.data_ptr() for k, v in d.items()}
        r.update(C=out.data_ptr() + 2 * off, N=c.N, R=0 if c.resA is None else c.resA.shape[1], b1=c.bits,
                 b2=3 if c.w2 is not None else 0, gs=c.gs)
        rows.append(r)
        off += c.N
    assert fx.qgemm_gemv_multi(x, _table(rows)) is None
    torch.cuda.synchronize()
    off = 0
    for c in cases:
        assert rel_err(out[:, off:off + c.N], c.oracle(x.cpu())) <= TOL, c.N
        off += c.N
    # gate + up + SiLU*mul
    g, u = Case(256, K, 128, 4, dt, seed=31), Case(256, K, 128, 4, dt, seed=32)
    bg, lg, bu, lu = g.blob.cuda(), g.lut.cuda(), u.blob.cuda(), u.lut.cuda()
    C = torch.empty(1, 256, dtype=dt, device="cuda")
    t = _table([dict(q1=bg.data_ptr(), lut1=lg.data_ptr(), N=256, b1=4, gs=128),
                dict(q1=bu.data_ptr(), lut1=lu.data_ptr(), N=256, b1=4, gs=128)])
    assert fx.qgemm_gemv_mlp(x, t, C) is C
    want = orc.silu_mul_fused(x.cpu().float() @ g.w1.t(), x.cpu().float() @ u.w1.t(), dt)
    assert rel_err(C, want) <= TOL


@gpu
def test_tables_whose_segments_carry_different_folds():
    K, dt = 4096, torch.bfloat16
    cases = [Case(n, K, 128, 4, dt, seed=40 + i, rotation_seed=7 + i, awq=i == 1) for i, n in enumerate((512, 256, 128))]
    x = cases[0].x(1).cuda()
    out = torch.full((1, sum(c.N for c in cases)), float("nan"), dtype=dt, device="cuda")
    keep, rows, off = [], [], 0
    for c in cases:
        d = dict(q1=c.blob.cuda(), lut1=c.lut.cuda(), signs=c.signs.cuda())
        if c.awq is not None:
            d["s"] = c.awq.cuda()
        keep.append(d)
        r = {k: v.data_ptr() for k, v in d.items()}
        r.update(C=out.data_ptr() + 2 * off, N=c.N, b1=4, gs=128)
        rows.append(r)
        off += c.N
    fx.qgemm_gemv_multi(x, _table(rows))
    torch.cuda.synchronize()
    off = 0
    for c in cases:
        assert rel_err(out[:, off:off + c.N], c.oracle(x.cpu())) <= TOL, c.N
        off += c.N
    # gate and up with different folds, then SiLU*mul
    g, u = cases[1], Case(256, K, 128, 4, dt, seed=50, rotation_seed=19)
    dg, du = keep[1], dict(q1=u.blob.cuda(), lut1=u.lut.cuda(), signs=u.signs.cuda())
    C = torch.empty(1, 256, dtype=dt, device="cuda")
    t = _table([dict({k: v.data_ptr() for k, v in dg.items()}, N=256, b1=4, gs=128),
                dict({k: v.data_ptr() for k, v in du.items()}, N=256, b1=4, gs=128)])
    assert fx.qgemm_gemv_mlp(x, t, C) is C
    want = orc.silu_mul_fused(g.oracle(x.cpu()).float(), u.oracle(x.cpu()).float(), dt)
    assert rel_err(C, want) <= 2 * TOL
