"""Case builders shared by the GPU parity tests: seeded synthetic projections,
their oracle (CPU) weights, and the product module on the device."""
from __future__ import annotations

import numpy as np
import torch

from conftest import load_pkg
from oracle import lut_linear_oracle as orc

pkg = load_pkg()
TOL = 1e-2      # max relative error bound on outputs (bf16/fp16 out, fp32 accumulate)


class Case:
    """One palettized projection: codes, palette(s), oracle weights, device module."""

    def __init__(self, N, K, gs, bits, dtype, seed, bits2=None, bias=False, residual=0,
                 n_groups=None, rotation_seed=None, awq=False, lut_std=0.02):
        self.N, self.K, self.gs, self.bits, self.dtype = N, K, gs, bits, dtype
        rng = np.random.default_rng(seed)
        g = torch.Generator().manual_seed(seed)
        ng = -(-N // gs) if n_groups is None else n_groups
        self.codes = rng.integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
        self.blob = torch.from_numpy(orc.pack_idxn(self.codes, bits))
        self.lut = (lut_std * torch.randn(ng, 1 << bits, generator=g)).sort(dim=1).values.to(dtype)
        self.w1 = orc.dequant_indices(self.codes, self.lut, gs, bits)
        kw = {}
        self.w2 = None
        if bits2 is not None:
            self.codes2 = rng.integers(0, 1 << bits2, size=(N, K), dtype=np.uint8)
            kw["indices2"] = torch.from_numpy(orc.pack_idxn(self.codes2, bits2))
            kw["lut2"] = (0.25 * lut_std * torch.randn(ng, 1 << bits2, generator=g)).to(dtype)
            kw["bitwidth2"] = bits2
            self.w2 = orc.dequant_indices(self.codes2, kw["lut2"], gs, bits2)
        self.bias = (0.1 * torch.randn(N, generator=g)).to(dtype) if bias else None
        self.resA = self.resB = None
        if residual:
            self.resA = (0.05 * torch.randn(N, residual, generator=g)).to(dtype)
            self.resB = (0.05 * torch.randn(residual, K, generator=g)).to(dtype)
            kw.update(resA=self.resA, resB=self.resB)
        self.signs = self.awq = None
        if rotation_seed is not None:
            kw.update(rotation_seed=rotation_seed, rotation_k=K)
            self.signs = orc.rotation_signs(K, rotation_seed)
            if awq:
                self.awq = (0.5 + torch.rand(K, generator=g)).float()
                kw.update(awq_scale=self.awq, fold_order="rotate_then_awq")
        self.kw = kw

    def module(self, device="cuda", reference=False):
        return pkg.PalettizedLinear(self.blob, self.lut, self.bits, self.gs, self.N, self.K,
                                    bias=self.bias, reference=reference, **self.kw).to(device)

    def x(self, M, seed=0, dtype=None):
        g = torch.Generator().manual_seed(1000 + seed)
        return torch.randn(M, self.K, generator=g).to(dtype or self.dtype)

    def oracle(self, x):
        return orc.linear_forward(x, self.w1, self.w2, resA=self.resA, resB=self.resB,
                                  bias=self.bias, rot_signs=self.signs, awq_scale=self.awq)


OBSERVED = {}    # test id -> largest max-relative error it measured (printed at the end of the run)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want| (the reference's rel-max form,
    src/scripts/test_qwen_weights.py:104-105); the largest value per test is kept so that the
    run's summary shows how far below the bound the kernels are."""
    import os
    e = orc.max_rel_err(got.detach().cpu().float(), want.detach().cpu().float())
    name = os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0]
    if e <= 5e-2 and e > OBSERVED.get(name, -1.0):     # larger values are deliberate contrasts
        OBSERVED[name] = e
    return e
