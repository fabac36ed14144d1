"""GPU parity of the PalettizedLinear module (kernel route and the GPU
restatement of the reference route) against outputs of the reference's own
forward stored in tests/golden/, and against the oracle on seeded cases."""
from __future__ import annotations

import importlib

import pytest
import torch

from helpers import TOL, Case, pkg, rel_err

pytestmark = pytest.mark.gpu


def _module_from_golden(golden, tag, reference):
    N, K, gs, b, M, b2, rank, has_bias, rot_seed, awq, x3d = (int(v) for v in golden.np(tag + "_meta"))
    kw = {}
    if b2 > 0:
        kw.update(indices2=torch.from_numpy(golden.np(tag + "_blob2")), lut2=golden.t(tag + "_lut2"),
                  bitwidth2=b2)
    if rank:
        kw.update(resA=golden.t(tag + "_resA"), resB=golden.t(tag + "_resB"))
    if has_bias:
        kw.update(bias=golden.t(tag + "_bias"))
    if rot_seed >= 0:
        kw.update(rotation_seed=rot_seed, rotation_k=K)
    if awq:
        kw.update(awq_scale=golden.t(tag + "_awq"), fold_order="rotate_then_awq")
    mod = pkg.PalettizedLinear(torch.from_numpy(golden.np(tag + "_blob")), golden.t(tag + "_lut"),
                               b, gs, N, K, reference=reference, **kw)
    return mod.cuda()


@pytest.mark.parametrize("case", range(7))
@pytest.mark.parametrize("reference", (False, True))
def test_forward_matches_reference_outputs(golden, case, reference):
    tag = f"fwd{case}"
    mod = _module_from_golden(golden, tag, reference)
    x, want = golden.t(tag + "_x"), golden.t(tag + "_y")
    got = mod(x.cuda())
    assert got.shape == want.shape and got.dtype == want.dtype
    assert rel_err(got, want) <= TOL


def test_reference_route_is_tight():
    # exact dequant + fp32 matmul: only the fp32 summation order differs from the CPU
    case = Case(512, 1024, 128, 4, torch.bfloat16, seed=8)
    x = case.x(4)
    got = case.module(reference=True)(x.cuda())
    assert rel_err(got, case.oracle(x)) <= 4e-3      # one bf16 ulp at the output scale


@pytest.mark.parametrize("M", (1, 2, 16))
def test_rotated_and_residual_modules(M):
    for case in (Case(256, 192, 64, 4, torch.float16, seed=31, rotation_seed=3),
                 Case(256, 4096, 128, 4, torch.bfloat16, seed=32, rotation_seed=7, awq=True),
                 Case(384, 256, 128, 3, torch.float16, seed=33, residual=8, bias=True, bits2=2)):
        x = case.x(M)
        assert rel_err(case.module()(x.cuda()), case.oracle(x)) <= TOL


def test_input_dtype_and_shape_handling():
    case = Case(256, 128, 128, 4, torch.bfloat16, seed=40)
    mod = case.module()
    x = case.x(6).reshape(2, 3, 128)
    y = mod(x.cuda())
    assert y.shape == (2, 3, 256) and y.dtype == torch.bfloat16
    assert rel_err(y.reshape(6, 256), case.oracle(x.reshape(6, 128))) <= TOL
    x32 = case.x(2, dtype=torch.float32)
    y32 = mod(x32.cuda())
    assert y32.dtype == torch.float32
    assert rel_err(y32, case.oracle(x32.bfloat16()).float()) <= TOL
    view = case.x(4)[:, :].cuda()[1:3]                  # an offset view
    assert rel_err(mod(view), case.oracle(view.cpu())) <= TOL
    assert mod(torch.empty(0, 128, dtype=torch.bfloat16, device="cuda")).shape == (0, 256)
    with pytest.raises(ValueError, match="feature dim"):
        mod(torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda"))


def test_logical_indices_and_weight_accessors():
    case = Case(256, 128, 64, 3, torch.float16, seed=41)
    mod = case.module()
    assert (mod._logical_indices_numpy() == case.codes).all()
    assert torch.equal(mod._quantized_weight().cpu(), case.w1)
    mod.drop_blob()
    x = case.x(1)
    assert rel_err(mod(x.cuda()), case.oracle(x)) <= TOL


def test_degenerate_shapes_follow_the_reference():
    # no rows: empty result; K == 0: zeros plus bias (kernel_streaming.cu:2363-2368)
    case = Case(128, 64, 128, 4, torch.bfloat16, seed=3, bias=True)
    mod = case.module()
    assert mod(torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda")).shape == (0, 128)
    assert mod(torch.zeros(2, 0, 64, dtype=torch.bfloat16, device="cuda")).shape == (2, 0, 128)
    lut = torch.zeros(1, 16, dtype=torch.bfloat16)
    bias = torch.arange(128, dtype=torch.bfloat16)
    k0 = pkg.PalettizedLinear(torch.zeros(0, dtype=torch.uint8), lut, 4, 128, 128, 0, bias=bias).cuda()
    y = k0(torch.zeros(3, 0, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (3, 128) and torch.equal(y.cpu(), bias.expand(3, 128))


def test_merged_launch_with_one_shared_rotation_and_residuals():
    K, dt = 512, torch.float16
    cases = [Case(n, K, 128, 4, dt, seed=40 + i, rotation_seed=9, residual=16, bias=(i == 1))
             for i, n in enumerate((256, 128, 384))]
    mods = [c.module() for c in cases]
    qkv = pkg.SplitQKV(*mods)
    x = cases[0].x(3)
    assert importlib.import_module(pkg.__name__ + ".palettized_modules")._mergeable(mods, x.cuda())
    got = qkv(x.cuda())
    torch.cuda.synchronize()
    want = torch.cat([c.oracle(x) for c in cases], dim=-1)
    assert got.shape == want.shape and rel_err(got, want) <= TOL
    # a different fold on one member: no merge, same result through the three modules
    odd = Case(128, K, 128, 4, dt, seed=50, rotation_seed=10)
    mixed = [mods[0], odd.module(), mods[2]]
    assert not importlib.import_module(pkg.__name__ + ".palettized_modules")._mergeable(mixed, x.cuda())
    got = pkg.SplitQKV(*mixed)(x.cuda())
    want = torch.cat([cases[0].oracle(x), odd.oracle(x), cases[2].oracle(x)], dim=-1)
    assert rel_err(got, want) <= TOL
