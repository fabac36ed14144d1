"""GPU parity of the decode GEMV (M <= 16) against the CPU oracle.

Tolerance: max |got - want| / max |want| <= 1e-2 (16-bit output, fp32 accumulate),
the bound the task states; dequantised weights are checked BIT-EXACT by feeding
one-hot activations through the same kernel (1.0 * w + zeros is exact in fp32).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, Case, pkg, rel_err
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib


def _run(case, x, split=0, workspace=None, flags=0):
    mod = case.module()
    mod._ensure_packed()
    xd = x.cuda()
    out = torch.full((x.shape[0], case.N), float("nan"), dtype=x.dtype, device="cuda")
    segs = L.make_segments([mod._segment_desc(out)])
    L.gemv_multi(xd, segs, 1, split=split, workspace=workspace, flags=flags)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("N,K,gs,bits,dtype,M", (
    (128, 64, 128, 4, torch.bfloat16, 1),
    (256, 256, 128, 4, torch.bfloat16, 1),
    (4096, 4096, 128, 4, torch.bfloat16, 1),       # the single-projection configuration
    (4096, 4096, 128, 4, torch.float16, 1),
    (1024, 4096, 64, 4, torch.bfloat16, 8),
    (1024, 4096, 64, 3, torch.bfloat16, 1),
    (512, 1024, 32, 4, torch.float16, 5),
    (512, 1024, 128, 3, torch.float16, 16),
    (384, 192, 64, 2, torch.bfloat16, 3),
    (256, 128, 256, 1, torch.bfloat16, 2),
    (2048, 12288, 128, 4, torch.bfloat16, 1),      # down-projection K
    (1024, 1024, 128, 4, torch.bfloat16, 9),
    (1024, 1024, 128, 4, torch.bfloat16, 16),
))
def test_gemv_matches_oracle(N, K, gs, bits, dtype, M):
    case = Case(N, K, gs, bits, dtype, seed=N + K + bits + M)
    x = case.x(M)
    got = _run(case, x)
    assert not torch.isnan(got.float()).any()
    assert rel_err(got, case.oracle(x)) <= TOL


@pytest.mark.parametrize("split", (1, 2, 3, 4, 5, 8, 12, 16))
def test_split_k_variants_agree(split):
    case = Case(512, 2048, 128, 4, torch.bfloat16, seed=split)
    x = case.x(4)
    want = case.oracle(x)
    ws = None
    nbytes = L.gemv_workspace_bytes(case.N, 4, split)
    if split > 8:
        assert nbytes > 0
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    else:
        assert nbytes == 0
    a = _run(case, x, split=split, workspace=ws)
    b = _run(case, x, split=split, workspace=ws)     # tickets reset themselves
    assert rel_err(a, want) <= TOL
    assert torch.equal(a, b)                         # deterministic, run to run


def test_workspace_too_small_is_refused():
    case = Case(256, 1024, 128, 4, torch.bfloat16, seed=1)
    with pytest.raises(L.LibraryError) as e:
        _run(case, case.x(1), split=16, workspace=torch.zeros(64, dtype=torch.uint8, device="cuda"))
    assert e.value.code == 4


@pytest.mark.parametrize("bits,gs,dtype", ((4, 128, torch.bfloat16), (4, 64, torch.float16),
                                           (3, 64, torch.bfloat16), (4, 32, torch.bfloat16),
                                           (2, 128, torch.float16), (1, 128, torch.bfloat16)))
def test_weights_through_the_kernel_are_bit_exact(bits, gs, dtype):
    # one-hot rows: y[m, :] = W[:, k_m] exactly
    N, K = 256, 192
    case = Case(N, K, gs, bits, dtype, seed=bits * 10 + gs)
    W = torch.empty(N, K, dtype=dtype)
    for k0 in range(0, K, 16):
        x = torch.zeros(16, K, dtype=dtype)
        x[torch.arange(16), k0 + torch.arange(16)] = 1.0
        W[:, k0:k0 + 16] = _run(case, x).cpu().t()
    assert torch.equal(W.float(), case.w1)


def test_row_group_clamp_and_bias():
    case = Case(512, 256, 128, 4, torch.bfloat16, seed=3, n_groups=2, bias=True)
    x = case.x(2)
    assert rel_err(_run(case, x), case.oracle(x)) <= TOL


def test_second_stream_mixed_widths():
    for (b1, b2) in ((4, 2), (3, 3), (4, 4), (4, 1)):
        case = Case(256, 512, 64, b1, torch.float16, seed=b1 * 7 + b2, bits2=b2)
        x = case.x(3)
        assert rel_err(_run(case, x), case.oracle(x)) <= TOL


def test_programmatic_launch_chain():
    # the same launches with the dependent-launch attribute give the same bits
    case = Case(1024, 1024, 128, 4, torch.bfloat16, seed=5)
    x = case.x(1)
    plain = _run(case, x)
    chained = [_run(case, x, flags=L.FLAG_PDL) for _ in range(4)]
    for c in chained:
        assert torch.equal(c, plain)


def test_merged_qkv_and_fused_mlp():
    dt = torch.bfloat16
    q, k, v = (Case(n, 512, 128, 4, dt, seed=s) for n, s in ((512, 1), (128, 2), (256, 3)))
    qkv = pkg.SplitQKV(q.module(), k.module(), v.module())
    x = q.x(1)
    got = qkv(x.cuda())
    want = torch.cat([c.oracle(x) for c in (q, k, v)], dim=-1)
    assert got.shape == (1, 896) and rel_err(got, want) <= TOL
    gate, up = Case(1024, 512, 128, 4, dt, seed=4, lut_std=0.05), Case(1024, 512, 128, 4, dt, seed=5)
    down = Case(512, 1024, 128, 4, dt, seed=6)
    mlp = pkg.FusedPalettizedMLP(gate.module(), up.module(), down.module(), torch.nn.SiLU())
    for M in (1, 8):
        x = gate.x(M)
        h = mlp.fused_gate_up(x.cuda())
        h_want = orc.silu_mul_fused(x.float() @ gate.w1.t(), x.float() @ up.w1.t(), dt)
        assert rel_err(h, h_want) <= TOL
        y = mlp(x.cuda())
        assert rel_err(y, orc.mlp_block_fused(x, gate.w1, up.w1, down.w1)) <= 2 * TOL
        assert rel_err(y, orc.mlp_block_unfused(x, gate.w1, up.w1, down.w1)) <= 2 * TOL


def test_mlp_block_shapes_of_the_9b_model():
    # gate/up 4096 -> 12288, down 12288 -> 4096, M = 1 and 8 (decode MLP block)
    dt = torch.bfloat16
    gate, up = Case(12288, 4096, 128, 4, dt, seed=21), Case(12288, 4096, 128, 4, dt, seed=22)
    down = Case(4096, 12288, 128, 4, dt, seed=23)
    mlp = pkg.FusedPalettizedMLP(gate.module(), up.module(), down.module(), torch.nn.SiLU())
    for M in (1, 8):
        x = gate.x(M)
        y = mlp(x.cuda())
        want = orc.mlp_block_fused(x, gate.w1, up.w1, down.w1)
        assert rel_err(y, want) <= 2 * TOL
        assert orc.cosine(y.cpu().float(), want.float()) >= 0.999


def test_persistent_plan_matches_per_launch_results():
    # a chain of jobs (merged heads, plain, fused gate/up, down on the fused output) in one
    # cooperative launch agrees with the separate launches to an output ulp, run after run
    dt = torch.bfloat16
    for M in (1, 4, 16):
        q, k, o = (Case(n, 1024, 128, 4, dt, seed=s) for n, s in ((512, 1), (128, 2), (1024, 3)))
        gate, up = Case(2048, 1024, 128, 4, dt, seed=4, lut_std=0.05), Case(2048, 1024, 128, 4, dt, seed=5)
        down = Case(1024, 2048, 64, 3, dt, seed=6)
        mods = {n: c.module() for n, c in dict(q=q, k=k, o=o, gate=gate, up=up, down=down).items()}
        for m in mods.values():
            m._ensure_packed()
        x = q.x(M).cuda()
        heads = torch.empty(M, 640, dtype=dt, device="cuda")
        obuf = torch.empty(M, 1024, dtype=dt, device="cuda")
        act = torch.empty(M, 2048, dtype=dt, device="cuda")
        y = torch.empty(M, 1024, dtype=dt, device="cuda")
        jobs = [
            dict(x=x, segs=[mods["q"]._segment_desc(heads, ldo=640), mods["k"]._segment_desc(heads[:, 512:], ldo=640)], dep=-1),
            dict(x=x, segs=[mods["o"]._segment_desc(obuf)], dep=0),
            dict(x=x, segs=[mods["gate"]._segment_desc(act), mods["up"]._segment_desc(None)],
                 epilogue=L.EPI_SILU_MUL, dep=1),
            dict(x=act, segs=[mods["down"]._segment_desc(y)], dep=2),
        ]
        want = []
        for j in jobs:
            L.gemv_multi(j["x"], L.make_segments(j["segs"]), len(j["segs"]), epilogue=j.get("epilogue", 0))
        torch.cuda.synchronize()
        want = [t.clone() for t in (heads, obuf, act, y)]
        plan = L.DecodePlan(jobs, M, dt, "cuda")
        for rep in range(3):
            for t in (heads, obuf, act, y):
                t.fill_(float("nan"))
            plan.run()
            torch.cuda.synchronize()
            plan.check_status()
            for got, w in zip((heads, obuf, act, y), want):
                assert rel_err(got, w) <= 5e-3     # same math, other K split points: one bf16 ulp
        assert rel_err(obuf, o.oracle(x.cpu())) <= TOL
        assert rel_err(y, down.oracle(act.cpu())) <= TOL


@pytest.mark.parametrize("M", (1, 3, 8))
def test_persistent_plan_of_row_range_jobs(M):
    # every job 4-bit and single-stream: the plan runs the row-range block body job after job.
    # Jobs wide enough to fill the SMs without a K split are laid out exactly as their single
    # launches, so their results are equal bit for bit; the narrow ones (a single launch splits
    # K over a cluster, a plan never does) agree to an output ulp.
    dt = torch.bfloat16
    q, k, o = (Case(n, 4096, 128, 4, dt, seed=s) for n, s in ((4096, 11), (1024, 12), (4096, 13)))
    gate, up = Case(4096, 4096, 128, 4, dt, seed=14, bias=True), Case(4096, 4096, 64, 4, dt, seed=15)
    down = Case(4096, 4096, 128, 4, dt, seed=16)
    small = Case(256, 1024, 64, 4, dt, seed=17)
    mods = {n: c.module() for n, c in dict(q=q, k=k, o=o, gate=gate, up=up, down=down, small=small).items()}
    for m in mods.values():
        m._ensure_packed()
    x = q.x(M).cuda()
    heads = torch.empty(M, 5120, dtype=dt, device="cuda")
    obuf = torch.empty(M, 4096, dtype=dt, device="cuda")
    act = torch.empty(M, 4096, dtype=dt, device="cuda")
    y = torch.empty(M, 4096, dtype=dt, device="cuda")
    tail = torch.empty(M, 256, dtype=dt, device="cuda")
    jobs = [
        dict(x=x, segs=[mods["q"]._segment_desc(heads, ldo=5120), mods["k"]._segment_desc(heads[:, 4096:], ldo=5120)], dep=-1),
        dict(x=x, segs=[mods["o"]._segment_desc(obuf)], dep=0),
        dict(x=x, segs=[mods["gate"]._segment_desc(act), mods["up"]._segment_desc(None)],
             epilogue=L.EPI_SILU_MUL, dep=1),
        dict(x=act, segs=[mods["down"]._segment_desc(y)], dep=2),
        dict(x=y[:, :1024], segs=[mods["small"]._segment_desc(tail)], dep=3),
    ]
    bufs = (heads, obuf, act, y, tail)
    for j in jobs:
        L.gemv_multi(j["x"], L.make_segments(j["segs"]), len(j["segs"]), epilogue=j.get("epilogue", 0))
    torch.cuda.synchronize()
    want = [t.clone() for t in bufs]
    plan = L.DecodePlan(jobs, M, dt, "cuda")
    assert plan.form == "rows"
    for rep in range(4):        # the counters return to zero by themselves
        for t in bufs:
            t.fill_(float("nan"))
        plan.run()
        torch.cuda.synchronize()
        plan.check_status()
        for i, (got, w) in enumerate(zip(bufs, want)):
            if i < 4:
                assert torch.equal(got, w), (rep, i)
            else:
                assert rel_err(got, w) <= 5e-3, (rep, i)
    assert rel_err(obuf, o.oracle(x.cpu())) <= TOL
    assert rel_err(y, down.oracle(act.cpu())) <= TOL
    assert L.lib().b200lut_device_status() == 0


# ---- fused low-rank residual ------------------------------------------------------------------
@pytest.mark.parametrize("M,K,R,dtype", ((1, 4096, 32, torch.bfloat16), (16, 1024, 256, torch.float16),
                                          (5, 192, 8, torch.bfloat16)))
def test_residual_projection_is_the_fp32_product(M, K, R, dtype):
    g = torch.Generator().manual_seed(K + R)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    resB = (0.05 * torch.randn(R, K, generator=g)).to(dtype).cuda()
    t = L.residual_project(x, resB)
    torch.cuda.synchronize()
    want = x.double() @ resB.double().t()
    assert rel_err(t.double().cpu(), want.cpu()) <= 1e-5
    t2 = L.residual_project(x, resB)
    assert torch.equal(t, t2)                       # fixed summation order


@pytest.mark.parametrize("N,K,gs,bits,dtype,M,R", (
    (4096, 4096, 128, 4, torch.bfloat16, 1, 32),    # the deployed recipe: 4-bit + rank 32
    (512, 1024, 64, 3, torch.float16, 16, 256),
    (256, 256, 128, 4, torch.bfloat16, 3, 8),
))
def test_fused_residual_matches_oracle(N, K, gs, bits, dtype, M, R):
    case = Case(N, K, gs, bits, dtype, seed=N + R, residual=R, bias=True)
    x = case.x(M)
    mod = case.module()
    assert mod._fusable_residual(M, dtype)
    got = mod(x.cuda())
    torch.cuda.synchronize()
    want = orc.linear_forward(x, case.w1, None, case.resA, case.resB, case.bias)
    assert rel_err(got.float().cpu(), want.float()) <= TOL
    # the residual really is in the kernel's output: without it the error is large
    plain = orc.linear_forward(x, case.w1, None, None, None, case.bias)
    assert rel_err(plain.float(), want.float()) > 5 * TOL


def test_fused_residual_in_a_gate_up_pair():
    N, K, R, M, dt = 512, 1024, 32, 2, torch.bfloat16
    gate, up = Case(N, K, 128, 4, dt, seed=1, residual=R), Case(N, K, 128, 4, dt, seed=2, residual=R)
    x = gate.x(M).cuda()
    g, u = gate.module(), up.module()
    resB = torch.cat([g.resB, u.resB], dim=0).contiguous()          # stacked first factors
    t = L.residual_project(x, resB)
    out = torch.empty(M, N, dtype=dt, device="cuda")
    descs = [g._segment_desc(out, res_t=t[:, :R]), u._segment_desc(None, res_t=t[:, R:])]
    L.gemv_multi(x, L.make_segments(descs), 2, epilogue=L.EPI_SILU_MUL)
    torch.cuda.synchronize()
    xf = x.float().cpu()
    gf = xf @ gate.w1.t() + (xf @ gate.resB.float().t()) @ gate.resA.float().t()
    uf = xf @ up.w1.t() + (xf @ up.resB.float().t()) @ up.resA.float().t()
    want = orc.silu_mul_fused(gf, uf, dt)
    assert rel_err(out.float().cpu(), want.float()) <= TOL
