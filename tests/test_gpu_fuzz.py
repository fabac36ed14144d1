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


def _merged_cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        M = int(rng.integers(17, 700))
        K = int(rng.choice([128, 192, 256, 512, 1024, 2048]))
        bits = int(rng.choice([1, 2, 3, 4]))
        gs = int(rng.choice([64, 128, 256]))
        Ns = tuple(256 * int(rng.integers(1, 5)) for _ in range(int(rng.integers(2, 5))))
        dtype = torch.bfloat16 if i % 2 == 0 else torch.float16
        out.append(pytest.param(M, K, bits, gs, Ns, dtype, bool(rng.integers(0, 2)),
                                id=f"{i}-M{M}-K{K}-b{bits}-gs{gs}-N{'+'.join(map(str, Ns))}"))
    return out


@pytest.mark.parametrize("M,K,bits,gs,Ns,dtype,bias", _merged_cases(16, 77))
def test_random_merged_prefill_launch_matches_oracle(M, K, bits, gs, Ns, dtype, bias):
    L = pkg._lib
    cases = [Case(N, K, gs, bits, dtype, seed=M + 7 * i, bias=bias) for i, N in enumerate(Ns)]
    mods = [c.module() for c in cases]
    x = cases[0].x(M)
    total = sum(Ns)
    out = torch.zeros(M, total, dtype=dtype, device="cuda")
    descs, off = [], 0
    for m in mods:
        descs.append(m._segment_desc(out[:, off:], ldo=total))
        off += m.N
    assert L.gemm_multi_ok(descs, K)
    L.gemm_multi(x.cuda(), L.make_segments(descs), len(descs))
    off = 0
    for c, m in zip(cases, mods):
        assert rel_err(out[:, off:off + m.N], c.oracle(x)) <= TOL
        off += m.N
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0
