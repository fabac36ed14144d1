"""GPU parity of the row-range decode GEMV (4-bit codes, M <= 8), selected with
B200LUT_FLAG_ROWS_KERNEL, against the CPU oracle and against the tile x K-split kernel.

Same bar as test_gpu_gemv: outputs within max |got - want| / max |want| <= 1e-2 (16-bit output,
fp32 accumulate); dequantised weights BIT-EXACT through one-hot activations; results
deterministic run to run. Shapes cover: one unit per block, several units and two palettes per
block, ranges that cross a segment boundary of a merged launch, the K split over a thread-block
cluster (few rows), K ranges that are and are not 64 chunks long (activation fragments in
registers / read from shared memory), ragged chunk counts, every batch size 1..8, both dtypes."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, Case, pkg, rel_err
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib
ROWS, TILE = L.FLAG_ROWS_KERNEL, L.FLAG_TILE_KERNEL


def _run(case, x, flags, mod=None):
    mod = mod or case.module()
    mod._ensure_packed()
    out = torch.full((x.shape[0], case.N), float("nan"), dtype=x.dtype, device="cuda")
    segs = L.make_segments([mod._segment_desc(out)])
    L.gemv_multi(x.cuda(), segs, 1, flags=flags)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("N,K,gs,dtype,M", (
    (128, 64, 128, torch.bfloat16, 1),          # one chunk: fifteen idle warps
    (256, 256, 128, torch.bfloat16, 1),         # four chunks: twelve idle warps
    (512, 1024, 32, torch.float16, 5),          # one palette per unit
    (1024, 4096, 64, torch.bfloat16, 8),        # 64 chunks: fragments in registers, M' = 8
    (4096, 4096, 128, torch.bfloat16, 1),       # the single-projection configuration
    (4096, 4096, 128, torch.float16, 1),
    (12288, 4096, 128, torch.bfloat16, 1),      # two or three units per block
    (12288, 4096, 64, torch.bfloat16, 2),       # up to three palettes per block
    (2048, 12288, 128, torch.bfloat16, 1),      # down-projection K, few rows: K split over a cluster of two
    (4096, 12288, 128, torch.bfloat16, 4),
    (640, 1856, 128, torch.bfloat16, 3),        # 29 chunks: ragged rounds, idle ring slots
    (9600, 2048, 128, torch.float16, 7),        # 32 chunks: half rounds
    (1024, 8192, 128, torch.bfloat16, 6),       # two full rounds per unit
    (32768, 1024, 128, torch.bfloat16, 8),      # seven units per block, each folded behind its last plane
    (20480, 1024, 64, torch.float16, 4),        # the same at M' = 4 with a palette per two units
))
def test_rows_kernel_matches_oracle(N, K, gs, dtype, M):
    case = Case(N, K, gs, 4, dtype, seed=N + K + M)
    x = case.x(M)
    got = _run(case, x, ROWS)
    assert not torch.isnan(got.float()).any()
    err = rel_err(got, case.oracle(x))
    print(f"rows kernel N={N} K={K} gs={gs} M={M}: max rel err {err:.2e}")
    assert err <= TOL
    assert torch.equal(got, _run(case, x, ROWS))            # deterministic, run to run
    assert rel_err(got, _run(case, x, TILE)) <= TOL           # the other kernel agrees
    assert L.lib().b200lut_device_status() == 0


@pytest.mark.parametrize("N,K,gs,dtype", ((256, 128, 128, torch.bfloat16), (4096, 256, 64, torch.float16),
                                          (12288, 64, 128, torch.bfloat16), (640, 4096, 32, torch.bfloat16)))
def test_rows_kernel_weights_are_bit_exact(N, K, gs, dtype):
    # x = e_k (one-hot rows): y[m, n] = W[n, k_m] exactly (1.0 * w + zeros in fp32, one rounding)
    case = Case(N, K, gs, 4, dtype, seed=3 * N + K)
    mod = case.module()
    ks = torch.tensor([0, 1, K // 2 + 3, K - 1, 17 % K, 63 % K, (K // 64 - 1) * 64, 5])
    x = torch.zeros(8, K, dtype=dtype)
    x[torch.arange(8), ks] = 1.0
    got = _run(case, x, ROWS, mod)
    want = case.w1[:, ks].t().to(dtype)
    assert torch.equal(got.cpu(), want)


def test_rows_kernel_merged_segments_bias_and_residual():
    # Q/K/V-like merge: three projections of different group sizes share x; unit ranges of the
    # blocks cross the segment boundaries; one segment carries a bias, one a fused residual
    K, M, dt = 4096, 3, torch.bfloat16
    cases = [Case(2048, K, 128, 4, dt, seed=1, bias=True), Case(1024, K, 64, 4, dt, seed=2),
             Case(4096, K, 128, 4, dt, seed=3, residual=16)]
    mods = [c.module() for c in cases]
    x = cases[0].x(M).cuda()
    total = sum(c.N for c in cases)
    for variant in (ROWS, TILE):
        out = torch.full((M, total), float("nan"), dtype=dt, device="cuda")
        descs, off = [], 0
        for c, m in zip(cases, mods):
            res_t = L.residual_project(x, m.resB) if m.has_residual() else None
            descs.append(m._segment_desc(out[:, off:], ldo=total, res_t=res_t))
            off += c.N
        L.gemv_multi(x, L.make_segments(descs), len(descs), flags=variant)
        torch.cuda.synchronize()
        off = 0
        for c in cases:
            assert rel_err(out[:, off:off + c.N], c.oracle(x.cpu())) <= TOL, (variant, c.N)
            off += c.N


@pytest.mark.parametrize("N,K,M", ((12288, 4096, 1), (12288, 4096, 8), (1024, 2048, 2), (256, 512, 1),
                                   (24576, 1024, 5), (12288, 4096, 3)))
def test_rows_kernel_fused_gate_up(N, K, M):
    dt = torch.bfloat16
    gate, up = Case(N, K, 128, 4, dt, seed=N + 1, bias=True), Case(N, K, 128, 4, dt, seed=N + 2)
    mg, mu = gate.module(), up.module()
    x = gate.x(M)
    want = orc.silu_mul_fused(x.float() @ gate.w1.t() + gate.bias.float(), x.float() @ up.w1.t(), dt)
    outs = []
    for variant in (ROWS, TILE):
        out = torch.full((M, N), float("nan"), dtype=dt, device="cuda")
        descs = [mg._segment_desc(out), mu._segment_desc(None)]
        L.gemv_multi(x.cuda(), L.make_segments(descs), 2, epilogue=L.EPI_SILU_MUL, flags=variant)
        torch.cuda.synchronize()
        assert rel_err(out, want) <= TOL, variant
        outs.append(out)
    assert rel_err(outs[0], outs[1]) <= TOL


def test_rows_kernel_leaves_other_widths_to_the_tile_kernel():
    # 3-bit codes and second streams are not served: the flag must not change their results
    case = Case(512, 1024, 128, 3, torch.bfloat16, seed=9)
    x = case.x(2)
    assert torch.equal(_run(case, x, ROWS), _run(case, x, TILE))
    two = Case(256, 512, 128, 4, torch.bfloat16, seed=10, bits2=2)
    x = two.x(1)
    assert torch.equal(_run(two, x, ROWS), _run(two, x, TILE))


@pytest.mark.parametrize("N,K,M,dtype,awq,exact", (
    (4096, 4096, 1, torch.bfloat16, False, True), (4096, 12288, 1, torch.float16, True, True),
    (12288, 4096, 8, torch.bfloat16, True, True), (256, 192, 2, torch.float16, False, True),
    # behind a separate transform the library policy gives this shape to the tile kernel (one unit
    # per block, K != 4096, M >= 2): same rotated rows, another summation order
    (4096, 12288, 3, torch.float16, True, False)))
def test_rotation_inside_the_launch_equals_the_separate_transform(N, K, M, dtype, awq, exact):
    """The module rotates its input inside the decode launch when it can (the reference's fused
    prologue, src/flute_extended/include/flute/gemv.cuh:305-351). Same butterfly, same rounding
    point: the outputs equal those behind a separate b200lut_fht launch bit for bit whenever the
    same decode kernel runs behind it."""
    import os
    case = Case(N, K, 128, 4, dtype, seed=N + K, rotation_seed=5, awq=awq)
    mod = case.module()
    x = case.x(M).cuda()
    assert mod._rotation_fuses(M, x.dtype)
    fused = mod(x)
    os.environ["FLUTE_NO_FHT_FUSE"] = "1"
    try:
        assert not mod._rotation_fuses(M, x.dtype)
        separate = mod(x)
    finally:
        del os.environ["FLUTE_NO_FHT_FUSE"]
    if exact:
        assert torch.equal(fused, separate)
    else:
        assert rel_err(fused, separate) <= 5e-3
    assert rel_err(fused, case.oracle(x.cpu())) <= TOL
    assert L.lib().b200lut_device_status() == 0


def test_gated_input_inside_the_launch():
    # down(silu(g) * u) with the product formed while the launch stages its rows
    dt, M, I, H = torch.bfloat16, 2, 12288, 4096
    case = Case(H, I, 128, 4, dt, seed=77)
    mod = case.module()
    mod._ensure_packed()
    g = torch.randn(M, I, generator=torch.Generator().manual_seed(1)).to(dt).cuda()
    u = torch.randn(M, I, generator=torch.Generator().manual_seed(2)).to(dt).cuda()
    out = torch.empty(M, H, dtype=dt, device="cuda")
    segs = L.make_segments([mod._segment_desc(out)])
    L.gemv_input(g, segs, 1, L.make_input(x_mul=u))
    act = L.silu_mul(g.clone(), u)
    want = torch.empty_like(out)
    L.gemv_multi(act, L.make_segments([mod._segment_desc(want)]), 1, flags=ROWS)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert rel_err(out, case.oracle(act.cpu())) <= TOL
    # shapes the fused form does not serve are refused, not silently served another way
    three = Case(256, 256, 128, 3, dt, seed=3).module()
    three._ensure_packed()
    o = torch.empty(1, 256, dtype=dt, device="cuda")
    with pytest.raises(L.LibraryError) as e:
        L.gemv_input(torch.zeros(1, 256, dtype=dt, device="cuda"), L.make_segments([three._segment_desc(o)]), 1,
                     L.make_input(x_mul=torch.zeros(1, 256, dtype=dt, device="cuda")))
    assert e.value.code == 2


# ---- a fold per segment ----------------------------------------------------------------------------
@pytest.mark.parametrize("Ns,K,M,dtype", (
    ((512, 256, 256), 4096, 1, torch.bfloat16),          # fewer units than SMs: one block per unit
    ((4096, 1024, 1024), 4096, 4, torch.float16),        # 192 units: the blocks are dealt to the segments
    ((2048, 4096, 512, 128), 12288, 2, torch.bfloat16),  # K = 8192 + 4096 values per fold
    ((256, 128), 192, 8, torch.bfloat16),                # K = 128 + 64: the butterfly in shared memory
))
def test_merged_launch_with_a_fold_per_segment(Ns, K, M, dtype):
    """Projections that share x but carry different folds run as ONE launch: every block
    rotates the rows with the fold of its segment (reference: the per-segment rotation of the
    merged kernels, src/flute_extended/src/kernel_gemv_multi.cu:101-334). Each segment's outputs
    equal those of its own launch behind its own transform, bit for bit when K is not split."""
    cases = []
    for i, n in enumerate(Ns):
        kind = i % 3          # rotated, rotated + AWQ scale, unrotated
        cases.append(Case(n, K, 128, 4, dtype, seed=300 + i + K, bias=bool(i & 1),
                          rotation_seed=None if kind == 2 else 11 + i, awq=kind == 1))
    mods = [c.module() for c in cases]
    x = cases[0].x(M).cuda()
    total = sum(Ns)
    out = torch.full((M, total), float("nan"), dtype=dtype, device="cuda")
    descs, off = [], 0
    for m in mods:
        m._ensure_packed()
        descs.append(m._segment_desc(out[:, off:], ldo=total))
        off += m.N
    inp = L.make_input(seg_folds=[m._fold(x.device) for m in mods])
    L.gemv_input(x, L.make_segments(descs), len(descs), inp)
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0
    off = 0
    for c, m in zip(cases, mods):
        got = out[:, off:off + c.N]
        off += c.N
        assert rel_err(got, c.oracle(x.cpu())) <= TOL
        if K == 4096:
            assert torch.equal(got, m(x))
    # the SiLU*mul epilogue shares one input between gate and up: refused with per-segment folds
    with pytest.raises(L.LibraryError):
        L.gemv_input(x, L.make_segments(descs[:2]), 2, inp, epilogue=L.EPI_SILU_MUL)


def test_module_layer_merges_projections_with_different_folds():
    K, M, dt = 4096, 1, torch.bfloat16
    q, k, v = (Case(n, K, 128, 4, dt, seed=400 + i, rotation_seed=21 + i, awq=i == 1)
               for i, n in enumerate((1024, 256, 256)))
    x = q.x(M)
    qkv = pkg.SplitQKV(q.module(), k.module(), v.module())
    assert pkg.palettized_modules._mergeable((qkv.q_proj, qkv.k_proj, qkv.v_proj), x.cuda(), per_segment=True)
    assert not pkg.palettized_modules._mergeable((qkv.q_proj, qkv.k_proj, qkv.v_proj), x.cuda())
    got = qkv(x.cuda())
    want = torch.cat([c.oracle(x) for c in (q, k, v)], dim=-1)
    assert rel_err(got, want) <= TOL
    gate, up, down = (Case(n, kk, 128, 4, dt, seed=410 + i, rotation_seed=31 + i)
                      for i, (n, kk) in enumerate(((1024, K), (1024, K), (K, 1024))))
    mlp = pkg.FusedPalettizedMLP(gate.module(), up.module(), down.module(), torch.nn.SiLU())
    got = mlp(x.cuda())
    act = (torch.nn.functional.silu(gate.oracle(x).float()) * up.oracle(x).float()).to(dt)
    assert rel_err(got, down.oracle(act)) <= 2 * TOL
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0
