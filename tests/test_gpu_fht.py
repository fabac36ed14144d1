"""GPU parity of the Hadamard rotation against the oracle and the reference-made
golden vectors. The butterfly is a fixed tree of fp32 adds, so equality is exact."""
from __future__ import annotations

import pytest
import torch

from helpers import pkg
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
fht = pkg.fht


@pytest.mark.parametrize("case", range(4))
def test_golden_forward_adjoint_awq(golden, case):
    M, K, seed = (int(v) for v in golden.np(f"fht{case}_meta"))
    x = golden.t(f"fht{case}_x").cuda()
    s = fht.rotation_signs(K, seed)
    assert torch.equal(fht.fht_apply(x, s).cpu(), golden.t(f"fht{case}_fwd"))
    assert torch.equal(fht.fht_adjoint(x, s).cpu(), golden.t(f"fht{case}_adj"))
    got = fht.fht_apply_awq(x, s, golden.t(f"fht{case}_scale"))
    assert torch.equal(got.cpu(), golden.t(f"fht{case}_awq"))


def test_golden_block128(golden):
    assert torch.equal(fht.fht_block(golden.t("fhtblk_x").cuda(), 128).cpu(), golden.t("fhtblk_y"))


@pytest.mark.parametrize("K", (64, 256, 4096, 12288, 6144, 192))
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16, torch.float32))
def test_seeded_rows_match_oracle(K, dtype):
    g = torch.Generator().manual_seed(K)
    x = torch.randn(5, K, generator=g).to(dtype)
    s = orc.rotation_signs(K, 17)
    assert torch.equal(fht.fht_apply(x.cuda(), s).cpu(), orc.fht_forward(x, s))
    assert torch.equal(fht.fht_adjoint(x.cuda(), s).cpu(), orc.fht_adjoint(x, s))


def test_in_place_and_3d_and_round_trip():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 3, 1024, generator=g)
    s = orc.rotation_signs(1024, 5)
    xd = x.cuda()
    y = fht.fht_apply(xd, s)
    assert y.shape == x.shape and torch.equal(y.cpu(), orc.fht_forward(x, s))
    back = fht.fht_adjoint(y, s)
    assert (back.cpu() - x).abs().max().item() < 1e-5       # the reference's own gate
    z = xd.clone()
    assert fht.fht_apply_(z, s) is z and torch.equal(z, y)
    T = fht.build_rotation_matrix(1024, 5)
    assert (y.cpu().reshape(-1, 1024) - x.reshape(-1, 1024) @ T).abs().max().item() < 1e-4


def test_prefill_block_rotation_full_size():
    # M = 2048 rows of K = 4096 in 128-point blocks: orthonormal (norm preserving),
    # an involution, and equal to the oracle on a sample of rows
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2048, 4096, generator=g).bfloat16()
    y = fht.fht_block(x.cuda(), 128)
    assert torch.equal(y[:8].cpu(), orc.fht_block(x[:8], 128))
    yf = fht.fht_block(x.cuda().float(), 128)
    assert torch.allclose(yf.norm(dim=1), x.float().norm(dim=1).cuda(), rtol=1e-4)
    assert (fht.fht_block(yf, 128) - x.cuda().float()).abs().max().item() < 1e-4


def test_autograd_is_the_adjoint():
    s = orc.rotation_signs(256, 9)
    x = torch.randn(3, 256, device="cuda", requires_grad=True)
    gy = torch.randn(3, 256, device="cuda")
    fht.fht_apply(x, s).backward(gy)
    assert torch.equal(x.grad.cpu(), orc.fht_adjoint(gy.cpu(), s))


def test_refusals():
    s = orc.rotation_signs(64, 0)
    with pytest.raises(RuntimeError, match="CUDA"):
        fht.fht_apply(torch.zeros(1, 64), s)
    with pytest.raises(ValueError, match="signs"):
        fht.fht_apply(torch.zeros(1, 128, device="cuda"), s)
    with pytest.raises(ValueError, match="backend"):
        fht.fht_apply(torch.zeros(1, 64, device="cuda"), s, backend="reference")
