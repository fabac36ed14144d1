"""Seeded random sweep of the module forward over shapes, widths, group sizes, batch sizes
and options, against the CPU oracle (max relative error <= 1e-2). Complements the hand-picked
cases: ragged token counts, K that is not a power of two, clamped palette rows, every route
(decode GEMV, tensor-core GEMM, 16-row slices), both dtypes."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, Case, pkg, rel_err

pytestmark = pytest.mark.gpu


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        N = 128 * int(rng.integers(1, 9))
        K = 64 * int(rng.integers(1, 25))
        gs = int(rng.choice([32, 64, 128, 256]))
        bits = int(rng.choice([1, 2, 3, 4], p=[0.1, 0.15, 0.25, 0.5]))
        dtype = torch.bfloat16 if rng.random() < 0.6 else torch.float16
        M = int(rng.choice([1, 2, 3, 5, 8, 13, 16, 17, 31, 64, 100, 129, 257, 300]))
        opts = dict(bias=bool(rng.random() < 0.4))
        if rng.random() < 0.25:
            opts["bits2"] = int(rng.choice([2, 3, 4]))
        if rng.random() < 0.3:
            opts["residual"] = int(rng.choice([8, 16, 32]))
        if rng.random() < 0.2:
            opts["rotation_seed"] = int(rng.integers(0, 100))
        if rng.random() < 0.15:                       # fewer palette rows than row groups: clamped
            opts["n_groups"] = max(1, -(-N // gs) - 1)
        out.append(pytest.param(N, K, gs, bits, dtype, M, opts, id=f"{i}-N{N}-K{K}-gs{gs}-b{bits}-M{M}"))
    return out


@pytest.mark.parametrize("N,K,gs,bits,dtype,M,opts", _cases(48, 20261125))
def test_random_module_forward_matches_oracle(N, K, gs, bits, dtype, M, opts):
    case = Case(N, K, gs, bits, dtype, seed=N * 7 + K + M, **opts)
    x = case.x(M)
    got = case.module()(x.cuda())
    torch.cuda.synchronize()
    assert got.shape == (M, N)
    assert rel_err(got, case.oracle(x)) <= TOL
    assert pkg._lib.lib().b200lut_device_status() == 0
