#!/usr/bin/env python3
"""Generate tests/golden/reference_vectors.npz by RUNNING the reference's own
Python code (its idxN packer, reference_dequant, PalettizedLinear(reference=True)
forward and fht reference) on seeded inputs.

Run where a checkout of pkhairkh/rag-cache-engineering-qwen35-9b-flute is
available:  python tests/golden/make_golden.py --reference <checkout>
The output file is committed; the tests only read it (the reference checkout is
not needed to run them). Floating tensors of 16-bit types are stored as their
raw uint16 bit patterns (key suffix "__bf16" / "__f16").
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch


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


def _sha(a) -> np.ndarray:
    a = a.contiguous().numpy() if torch.is_tensor(a) else np.ascontiguousarray(a)
    return np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8).copy()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its own Python modules are imported from it)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "reference_vectors.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src", "scripts"))
    sys.path.insert(0, os.path.join(args.reference, "src", "flute_extended"))
    import palettized_modules as pm          # the reference runtime layer
    idxn = pm._get_idxn()                    # the reference idxN packer
    fht = pm._get_fht()                      # the reference FHT module
    torch.set_num_threads(1)                 # fixed fp32 summation order

    out = {}
    assert idxn.self_test()

    # 1. idxN pack: the self-test shapes and seed (idxN.py:311-329). Small
    #    shapes are stored whole, large ones as sha256 of the blob.
    rng = np.random.default_rng(0)
    for b in (1, 2, 3, 4):
        for (N, K) in ((128, 64), (256, 128), (384, 192), (1024, 512)):
            idx = rng.integers(0, 1 << b, size=(N, K), dtype=np.uint8)
            blob = idxn.pack_idxn(idx, b)
            tag = f"idxn_b{b}_{N}x{K}"
            if N * K <= 256 * 128:
                out[tag + "_idx"] = idx
                out[tag + "_blob"] = blob
            else:
                out[tag + "_idx_sha"] = _sha(idx)
                out[tag + "_blob_sha"] = _sha(blob)

    # 2. reference_dequant, bf16 and fp16 palettes, 3 and 4 bit, with a short
    #    LUT grid (row-group clamp) in one case.
    for case, (N, K, gs, b, dt, ng) in enumerate((
            (128, 64, 32, 4, torch.bfloat16, None),
            (256, 128, 64, 3, torch.float16, None),
            (256, 64, 128, 4, torch.float16, 1),
            (128, 128, 128, 2, torch.bfloat16, None))):
        g = torch.Generator().manual_seed(100 + case)
        r = np.random.default_rng(100 + case)
        idx = r.integers(0, 1 << b, size=(N, K), dtype=np.uint8)
        blob = idxn.pack_idxn(idx, b)
        groups = (N // gs) if ng is None else ng
        lut = (0.02 * torch.randn(groups, 1 << b, generator=g)).sort(dim=1).values.to(dt)
        W = pm.reference_dequant(torch.from_numpy(blob), lut, N, K, gs, b)
        tag = f"deq{case}"
        out[tag + "_meta"] = np.array([N, K, gs, b, groups], dtype=np.int64)
        out[tag + "_blob"] = blob
        _store(out, tag + "_lut", lut)
        _store(out, tag + "_W", W)

    # 3. forward of PalettizedLinear(reference=True)
    def module_case(tag, N, K, gs, b, dt, M, seed, b2=None, residual=0, bias=False,
                    rotation_seed=None, awq=False, x3d=False):
        g = torch.Generator().manual_seed(seed)
        r = np.random.default_rng(seed)
        idx = r.integers(0, 1 << b, size=(N, K), dtype=np.uint8)
        blob = torch.from_numpy(idxn.pack_idxn(idx, b))
        lut = (0.02 * torch.randn(N // gs, 1 << b, generator=g)).sort(dim=1).values.to(dt)
        kw = {}
        if b2 is not None:
            idx2 = r.integers(0, 1 << b2, size=(N, K), dtype=np.uint8)
            kw["indices2"] = torch.from_numpy(idxn.pack_idxn(idx2, b2))
            kw["lut2"] = (0.005 * torch.randn(N // gs, 1 << b2, generator=g)).to(dt)
            kw["bitwidth2"] = b2
            out[tag + "_blob2"] = kw["indices2"].numpy()
            _store(out, tag + "_lut2", kw["lut2"])
        if residual:
            kw["resA"] = (0.05 * torch.randn(N, residual, generator=g)).to(dt)
            kw["resB"] = (0.05 * torch.randn(residual, K, generator=g)).to(dt)
            _store(out, tag + "_resA", kw["resA"])
            _store(out, tag + "_resB", kw["resB"])
        if bias:
            kw["bias"] = (0.1 * torch.randn(N, generator=g)).to(dt)
            _store(out, tag + "_bias", kw["bias"])
        if rotation_seed is not None:
            kw["rotation_seed"] = rotation_seed
            kw["rotation_k"] = K
        if awq:
            kw["awq_scale"] = (0.5 + torch.rand(K, generator=g)).float()
            kw["fold_order"] = "rotate_then_awq"
            _store(out, tag + "_awq", kw["awq_scale"])
        mod = pm.PalettizedLinear(blob, lut, b, gs, N, K, reference=True, **kw)
        shape = (2, M // 2, K) if x3d else (M, K)
        x = torch.randn(*shape, generator=g).to(dt)
        with torch.no_grad():
            y = mod(x)
        out[tag + "_meta"] = np.array([N, K, gs, b, M, -1 if b2 is None else b2, residual,
                                       int(bias), -1 if rotation_seed is None else rotation_seed,
                                       int(awq), int(x3d)], dtype=np.int64)
        out[tag + "_blob"] = blob.numpy()
        _store(out, tag + "_lut", lut)
        _store(out, tag + "_x", x)
        _store(out, tag + "_y", y)
        if mod.rot_signs is not None:
            _store(out, tag + "_signs", mod.rot_signs)

    module_case("fwd0", 128, 64, 32, 4, torch.float16, 3, 0, residual=8)       # test_finetune.py:96-129 shape
    module_case("fwd1", 128, 128, 32, 4, torch.float16, 2, 1, b2=2)            # two-stream (4,2) head
    module_case("fwd2", 256, 256, 128, 4, torch.bfloat16, 1, 2)                # bf16 decode row
    module_case("fwd3", 256, 192, 64, 3, torch.bfloat16, 16, 3, bias=True)     # 3-bit, bias
    module_case("fwd4", 128, 192, 64, 4, torch.float16, 1, 4, rotation_seed=3)  # rotated, K = 128 + 64
    module_case("fwd5", 128, 256, 128, 4, torch.bfloat16, 4, 5, rotation_seed=11, awq=True, x3d=True)
    module_case("fwd6", 384, 512, 128, 4, torch.bfloat16, 8, 6, b2=3, residual=16, bias=True)

    # 4. rotation_signs: full vectors for the K the projections use
    for (K, seed) in ((64, 0), (1024, 7), (1024, 42), (4096, 0), (12288, 3)):
        out[f"signs_K{K}_s{seed}"] = fht.rotation_signs(K, seed).to(torch.int8).numpy()

    # 5. fht reference forward/adjoint/awq, incl. a two-segment K, and the
    #    explicit-matrix agreement the reference tests gate on
    for case, (M, K, seed, dt) in enumerate(((8, 1024, 7, torch.float32),
                                             (3, 192, 1, torch.bfloat16),
                                             (2, 4096, 0, torch.float16),
                                             (1, 12288, 3, torch.bfloat16))):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(M, K, generator=g).to(dt)
        s = fht.rotation_signs(K, seed)
        tag = f"fht{case}"
        out[tag + "_meta"] = np.array([M, K, seed], dtype=np.int64)
        _store(out, tag + "_x", x)
        _store(out, tag + "_fwd", fht.fht_reference(x, s))
        _store(out, tag + "_adj", fht.fht_reference_adjoint(x, s))
        sc = (0.5 + torch.rand(K, generator=g)).float()
        _store(out, tag + "_scale", sc)
        _store(out, tag + "_awq", fht.fht_apply_awq(x, s, sc, backend="reference"))
    x = torch.randn(4, 512, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    _store(out, "fhtblk_x", x)
    _store(out, "fhtblk_y", fht.fht_reference(x.reshape(-1, 128), torch.ones(128)).reshape_as(x))

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
