#!/usr/bin/env python3
"""Generate tests/golden/embedding_vectors.npz by RUNNING the reference's own
PalettizedEmbedding.forward (src/scripts/palettized_modules.py:1979-2335) on seeded
tables and ids: one and two code streams, the low-rank residual, the tied-head
rotation (rows un-rotated through the adjoint Hadamard transform), fp16 and bf16
palettes, 1..4-bit codes.

Run where a checkout of pkhairkh/rag-cache-engineering-qwen35-9b-flute is
available:  python tests/golden/make_embedding_golden.py --reference <checkout>
The output file is committed; the tests only read it. 16-bit floating tensors are
stored as raw uint16 bit patterns (key suffix "__bf16" / "__f16").
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

CASES = (
    # name,  N,   K,  gs, bits, dtype,          bits2, rank, rot_seed, ids shape
    ("e1", 256, 128, 64, 4, torch.float16, None, 0, None, (9,)),
    ("e2", 384, 192, 128, 3, torch.bfloat16, None, 0, None, (2, 5)),
    ("e3", 256, 256, 32, 4, torch.float16, 2, 0, None, (7,)),
    ("e4", 128, 64, 128, 2, torch.float16, 4, 8, None, (3, 2)),
    ("e5", 512, 256, 128, 4, torch.float16, None, 16, 5, (6,)),
    ("e6", 256, 192, 64, 1, torch.bfloat16, 3, 0, 9, (4,)),
    ("e7", 1024, 512, 128, 4, torch.bfloat16, None, 0, 21, (2, 3)),
)


def _store(out, key, t):
    if torch.is_tensor(t):
        if t.dtype == torch.bfloat16:
            out[key + "__bf16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
        elif t.dtype == torch.float16:
            out[key + "__f16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
        else:
            out[key] = t.contiguous().numpy()
    else:
        out[key] = np.asarray(t)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its own Python modules are imported from it)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "embedding_vectors.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src", "scripts"))
    sys.path.insert(0, os.path.join(args.reference, "src", "flute_extended"))
    import palettized_modules as pm
    idxn = pm._get_idxn()
    torch.set_num_threads(1)

    out = {}
    for seed, (name, N, K, gs, bits, dtype, bits2, rank, rot, shape) in enumerate(CASES):
        rng = np.random.default_rng(100 + seed)
        g = torch.Generator().manual_seed(200 + seed)
        ng = -(-N // gs)
        codes = rng.integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
        lut = (0.02 * torch.randn(ng, 1 << bits, generator=g)).to(dtype)
        kw = {}
        _store(out, f"{name}_codes", codes)
        _store(out, f"{name}_lut", lut)
        if bits2 is not None:
            codes2 = rng.integers(0, 1 << bits2, size=(N, K), dtype=np.uint8)
            lut2 = (0.005 * torch.randn(ng, 1 << bits2, generator=g)).to(dtype)
            kw.update(indices2=torch.from_numpy(idxn.pack_idxn(codes2, bits2)), lut2=lut2,
                      bitwidth2=bits2)
            _store(out, f"{name}_codes2", codes2)
            _store(out, f"{name}_lut2", lut2)
        if rank:
            resA = (0.05 * torch.randn(N, rank, generator=g)).to(dtype)
            resB = (0.05 * torch.randn(rank, K, generator=g)).to(dtype)
            kw.update(resA=resA, resB=resB)
            _store(out, f"{name}_resA", resA)
            _store(out, f"{name}_resB", resB)
        if rot is not None:
            kw.update(rotation_seed=rot, rotation_k=K)
        mod = pm.PalettizedEmbedding(torch.from_numpy(idxn.pack_idxn(codes, bits)), lut, bits, gs,
                                     N, K, **kw)
        ids = torch.from_numpy(rng.integers(0, N, size=shape, dtype=np.int64))
        ids.view(-1)[0] = N - 1                       # the last row of the table
        ids.view(-1)[-1] = 0
        with torch.no_grad():
            y = mod(ids)
        assert y.shape == tuple(shape) + (K,) and y.dtype == dtype
        _store(out, f"{name}_ids", ids)
        _store(out, f"{name}_out", y)
        out[f"{name}_meta"] = np.array([N, K, gs, bits, bits2 or 0, rank, -1 if rot is None else rot],
                                       dtype=np.int64)
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
