"""The hybrid-palettization grid at the model's own projection shapes: {4096 x 4096,
12288 x 4096} x code width {3, 4} x group size {64, 128} x batch {1, 16, 128}, through the
module forward (decode GEMV at M <= 16, tensor-core GEMM at M = 128).

The codes are drawn on the device and the oracle side is bounded by sampling: the kernel's own
code export (bit-exact against the oracle in test_gpu_layout) gives the codes of 512 weight
rows spread over the matrix, including the first and last tile and a palette-group boundary;
their outputs are recomputed on the CPU with the reference route's arithmetic (palette lookup,
fp32 matmul, one rounding; src/scripts/palettized_modules.py:125-162, 1241-1251) and compared
within the output tolerance. The observed maximum is printed so a drift shows before it fails."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, pkg, rel_err

pytestmark = pytest.mark.gpu
L = pkg._lib


def _sample_rows(N: int) -> torch.Tensor:
    tiles = sorted({0, 1, (N // 128) // 3, (N // 128) - 1})
    return torch.cat([torch.arange(t * 128, t * 128 + 128) for t in tiles])


@pytest.mark.parametrize("N", (4096, 12288))
@pytest.mark.parametrize("bits", (3, 4))
@pytest.mark.parametrize("gs", (64, 128))
def test_hybrid_grid_at_model_shapes(N, bits, gs):
    K = 4096
    seed = 4000 + N // 128 + 8 * bits + gs
    blob = pkg.synthetic.random_blob_on_device(N, K, bits, seed, "cuda")
    lut = pkg.synthetic.make_lut(N // gs, bits, torch.bfloat16, seed)
    mod = pkg.PalettizedLinear(blob, lut.cuda(), bits, gs, N, K).cuda()
    rows = _sample_rows(N)
    mod._ensure_packed()
    codes = L.unpack_codes(mod._packed, N, K, bits)[rows.cuda()].cpu().numpy().astype(np.int64)
    w = torch.empty(len(rows), K)
    for j, r in enumerate(rows.tolist()):
        w[j] = lut[r // gs].float()[torch.from_numpy(codes[j])]
    worst = {}
    for M in (1, 16, 128):
        x = pkg.synthetic.make_x(M, K, torch.bfloat16, seed + M)
        got = mod(x.cuda())
        want = (x.float() @ w.t()).to(torch.bfloat16)
        worst[M] = rel_err(got[:, rows.cuda()], want)
    print(f"hybrid grid N={N} bits={bits} gs={gs}: max rel err {worst}")
    assert max(worst.values()) <= TOL, worst
    assert L.lib().b200lut_device_status() == 0
