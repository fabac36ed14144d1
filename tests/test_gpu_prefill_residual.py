"""GPU parity of the low-rank residual inside the prefill GEMM (M > 16).

t = x @ resB^T comes from b200lut_residual_project_rows (rounded once to the compute dtype, as
the reference route rounds it), then t and the projection's resA rows ride the tensor-core
launch as extra k-blocks of the same accumulator. Tolerance against the CPU oracle:
max |got - want| / max |want| <= 1e-2."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, Case, pkg, rel_err
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0, "a bounded wait ran out inside a kernel"


@pytest.mark.parametrize("M,K,R,dtype", (
    (64, 4096, 32, torch.bfloat16), (2048, 4096, 32, torch.bfloat16), (37, 192, 40, torch.float16),
    (300, 1024, 96, torch.bfloat16), (17, 64, 8, torch.float16), (129, 12288, 32, torch.bfloat16),
))
def test_projection_rows_is_the_rounded_product_with_zero_padding(M, K, R, dtype):
    g = torch.Generator().manual_seed(K + R + M)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    resB = (0.05 * torch.randn(R, K, generator=g)).to(dtype).cuda()
    cols = L.residual_block_cols(R)
    t = torch.full((M, cols), float("nan"), dtype=dtype, device="cuda")
    L.residual_project_rows(x, resB, out=t)
    torch.cuda.synchronize()
    want = (x.double() @ resB.double().t()).cpu()
    # one rounding of an fp32 sum: half an ulp of the 16-bit type
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert rel_err(t[:, :R].double().cpu(), want) <= ulp
    assert cols % 64 == 0 and torch.count_nonzero(t[:, R:]) == 0
    t2 = L.residual_project_rows(x, resB)
    assert torch.equal(t, t2)                       # fixed summation order


@pytest.mark.parametrize("N,K,gs,bits,dtype,M,R", (
    (4096, 4096, 128, 4, torch.bfloat16, 64, 32),    # the deployed recipe at a short prompt
    (1024, 1024, 64, 3, torch.float16, 100, 40),     # rank not a multiple of 16
    (512, 2048, 128, 4, torch.bfloat16, 300, 96),    # two residual k-blocks per tile
    (256, 256, 128, 2, torch.bfloat16, 17, 8),
    (12288, 1024, 128, 4, torch.bfloat16, 512, 32),  # 192 tiles: the cut tiles carry the residual too
))
def test_fused_prefill_residual_matches_oracle(N, K, gs, bits, dtype, M, R):
    case = Case(N, K, gs, bits, dtype, seed=N + R + M, residual=R, bias=True)
    x = case.x(M)
    mod = case.module()
    assert mod._fusable_residual(M, dtype)
    got = mod(x.cuda())
    torch.cuda.synchronize()
    want = case.oracle(x)
    assert rel_err(got, want) <= TOL
    plain = orc.linear_forward(x, case.w1, None, None, None, case.bias)
    assert rel_err(plain, want) > 5 * TOL           # the residual really is in the output


def test_residual_columns_through_the_gemm_are_exact():
    # zero palettes and one-hot t rows would need a crafted x; instead: zero codes' palette
    # entries (all-zero LUT) leave y = t @ resA^T, and x = rows of an identity picks resB
    # columns exactly, so the launch must reproduce round(resB[:, k]) @ resA^T
    N, K, R, dt = 256, 128, 16, torch.bfloat16
    case = Case(N, K, 128, 4, dt, seed=5, residual=R)
    lut0 = torch.zeros_like(case.lut)
    mod = pkg.PalettizedLinear(case.blob, lut0, 4, 128, N, K, resA=case.resA, resB=case.resB).cuda()
    x = torch.eye(K, dtype=dt)
    got = mod(x.cuda()).float().cpu()                # [K, N]
    want = (case.resB.float().t() @ case.resA.float().t())
    assert rel_err(got, want.to(dt)) <= 2.0 ** -8


def test_prefill_shape_of_the_9b_model_with_rank_32_sampled():
    N, K, M, gs, R = 12288, 4096, 2048, 128, 32
    g = torch.Generator().manual_seed(9)
    blob = pkg.synthetic.random_blob_on_device(N, K, 4, 177, "cuda")
    lut = pkg.synthetic.make_lut(N // gs, 4, torch.bfloat16, 177)
    resA = (0.05 * torch.randn(N, R, generator=g)).to(torch.bfloat16)
    resB = (0.05 * torch.randn(R, K, generator=g)).to(torch.bfloat16)
    mod = pkg.PalettizedLinear(blob, lut.cuda(), 4, gs, N, K, resA=resA.cuda(), resB=resB.cuda()).cuda()
    x = pkg.synthetic.make_x(M, K, torch.bfloat16, 178)
    got = mod(x.cuda())
    rows = torch.cat([torch.arange(t * 128, t * 128 + 128) for t in (0, 41, 77, 95)])
    codes = L.unpack_codes(mod._packed, N, K, 4)[rows.cuda()].cpu().numpy()
    w = torch.empty(len(rows), K)
    for j, r in enumerate(rows.tolist()):
        w[j] = lut[r // gs].float()[torch.from_numpy(codes[j].astype(np.int64))]
    want = orc.linear_forward(x, w, None, resA[rows], resB, None)
    assert rel_err(got[:, rows.cuda()], want) <= TOL


def test_two_stream_prefill_carries_the_residual_in_its_second_launch():
    case = Case(512, 1024, 128, 3, torch.bfloat16, seed=31, bits2=2, residual=32, bias=True)
    x = case.x(200)
    mod = case.module()
    assert mod._fusable_residual(200, torch.bfloat16)
    assert rel_err(mod(x.cuda()), case.oracle(x)) <= TOL


def test_merged_prefill_launches_carry_each_projections_residual():
    K, M, dt = 1024, 96, torch.bfloat16
    q, k, v = (Case(n, K, 128, 4, dt, seed=50 + i, residual=r, bias=bool(i))
               for i, (n, r) in enumerate(((512, 32), (256, 0), (256, 72))))
    x = q.x(M)
    qkv = pkg.SplitQKV(q.module(), k.module(), v.module())
    got = qkv(x.cuda())
    want = torch.cat([c.oracle(x) for c in (q, k, v)], dim=-1)
    assert rel_err(got, want) <= TOL
    gate, up, down = (Case(n, kk, 128, 4, dt, seed=60 + i, residual=32)
                      for i, (n, kk) in enumerate(((768, K), (768, K), (K, 768))))
    mlp = pkg.FusedPalettizedMLP(gate.module(), up.module(), down.module(), torch.nn.SiLU())
    got = mlp(x.cuda())
    act = (torch.nn.functional.silu(gate.oracle(x).float()) * up.oracle(x).float()).to(dt)
    assert rel_err(got, down.oracle(act)) <= 2 * TOL     # two roundings of the activation on the way


def test_a_residual_prefill_forward_launches_no_library_gemm():
    torch.profiler  # noqa: B018  (the profiler needs CUPTI; skip where it cannot start)
    case = Case(1024, 1024, 128, 4, torch.bfloat16, seed=3, residual=32, bias=True)
    mod = case.module()
    x = case.x(256).cuda()
    mod(x)
    torch.cuda.synchronize()
    try:
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
            mod(x)
            torch.cuda.synchronize()
        names = [e.name for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    except Exception as exc:       # pragma: no cover
        pytest.skip(f"profiler unavailable: {exc}")
    if not names:
        pytest.skip("the profiler recorded no kernels")
    assert any("residual_rows_kernel" in n for n in names)
    assert any("gemm_tc_persistent_kernel" in n for n in names)
    foreign = [n for n in names if any(s in n.lower() for s in ("cutlass", "cublas", "gemm", "gemv", "xmma"))
               and "b200lut" not in n]
    assert not foreign, foreign
