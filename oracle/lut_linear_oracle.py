"""CPU oracle for the idxN LUT-palettized linear layer.

TEST INFRASTRUCTURE ONLY. This module is the checker, never the product:
only the test-suite, the smoke entry and the benchmark's CPU-baseline /
reference arm may import it. The CUDA library never routes through it.

It restates, in numpy / CPU torch, the arithmetic of the reference project
(pkhairkh/rag-cache-engineering-qwen35-9b-flute). Each function cites the
reference file:line it follows. Parity is PINNED: tests/golden/ holds outputs
of the reference's own Python code (its idxN packer, its reference_dequant,
its PalettizedLinear(reference=True).forward, its PalettizedEmbedding.forward and its
fht_reference), made by tests/golden/make_golden.py and
tests/golden/make_embedding_golden.py, and tests/test_oracle_golden.py checks every
function here against them bit for bit.

Conventions: indices are the logical [N, K] uint8 code matrix; a "blob" is the
idxN byte stream; LUT is [ceil(N/gs), 2**bits]; W[n, k] = LUT[n // gs, idx[n, k]].
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

ROWS_PER_TILE = 128   # src/flute_extended/flute_extended/idxN.py:85
K_PER_TILE = 64       # idxN.py:86
THREADS_PER_TILE = 64  # idxN.py:89
ELEMS_PER_THREAD = 128  # idxN.py:87 (64 k-pairs)


# --------------------------------------------------------------------------- #
# idxN blob <-> logical indices (src/flute_extended/flute_extended/idxN.py)
# --------------------------------------------------------------------------- #

def idxn_coordinates() -> Tuple[np.ndarray, np.ndarray]:
    """Tile-local (row, k) of element e of thread-chunk th, shape [64, 128].

    Follows the normative layout text of idxN.py:37-55 and the loop nest of
    idxN.py:124-155: element e = 2*p + j with p = kt*16 + v*4 + d*2 + s2,
    row = wx*64 + v*16 + d*8 + (lane >> 2), k = kt*16 + 2*(lane & 3) + 8*s2 + j,
    thread th = wx*32 + lane. Written here as closed-form integer arithmetic on
    an (th, e) grid instead of the reference's nested loops.
    """
    th, e = np.meshgrid(np.arange(THREADS_PER_TILE), np.arange(ELEMS_PER_THREAD),
                        indexing="ij")
    wx, lane = th // 32, th % 32
    j, p = e % 2, e // 2
    s2, d, v, kt = p % 2, (p // 2) % 2, (p // 4) % 4, p // 16
    row = wx * 64 + v * 16 + d * 8 + (lane >> 2)
    col = kt * 16 + 2 * (lane & 3) + 8 * s2 + j
    return row.astype(np.int64), col.astype(np.int64)


def _check_shape(N: int, K: int, bits: int) -> None:
    # idxN.py:95-108 (same refusals: width in 1..4, N % 128, K % 64)
    if int(bits) not in (1, 2, 3, 4):
        raise ValueError(f"idxN supports bit widths (1, 2, 3, 4), got bits={bits}")
    if N % ROWS_PER_TILE != 0:
        raise ValueError(f"idxN layout requires N % 128 == 0, got N={N}")
    if K % K_PER_TILE != 0:
        raise ValueError(f"idxN layout requires K % 64 == 0, got K={K}")


def pack_idxn(indices: np.ndarray, bits: int) -> np.ndarray:
    """Logical [N, K] codes -> idxN blob (idxN.py:235-264).

    Every width is an LSB-first bit stream of `bits`-bit fields inside each
    16*bits-byte thread chunk (idxN.py:158-192: the b=3 "24-bit little-endian
    group of 8 fields" is the same stream), so one little-endian packbits
    serves all widths.
    """
    idx = np.ascontiguousarray(indices, dtype=np.uint8)
    if idx.ndim != 2:
        raise ValueError(f"expected a 2-D index matrix, got shape {idx.shape}")
    N, K = idx.shape
    _check_shape(N, K, bits)
    if idx.size and int(idx.max()) >= (1 << bits):
        raise ValueError(f"idx{bits} indices must be < {1 << bits}, got max {int(idx.max())}")
    row, col = idxn_coordinates()
    T, G = N // ROWS_PER_TILE, K // K_PER_TILE
    tiles = idx.reshape(T, ROWS_PER_TILE, G, K_PER_TILE).transpose(0, 2, 1, 3)
    elems = tiles[:, :, row, col]                               # [T, G, 64, 128]
    planes = (elems[..., None] >> np.arange(bits, dtype=np.uint8)) & 1
    stream = planes.reshape(T, G, THREADS_PER_TILE, ELEMS_PER_THREAD * bits)
    return np.packbits(stream, axis=-1, bitorder="little").reshape(-1)


def unpack_idxn(blob: np.ndarray, N: int, K: int, bits: int) -> np.ndarray:
    """idxN blob -> logical [N, K] codes (idxN.py:267-291)."""
    _check_shape(N, K, bits)
    blob = np.ascontiguousarray(blob, dtype=np.uint8).reshape(-1)
    expected = N * K * bits // 8
    if blob.size != expected:
        raise ValueError(f"idx{bits} blob has {blob.size} bytes, expected N*K*{bits}/8 = "
                         f"{expected} (N={N}, K={K})")
    row, col = idxn_coordinates()
    T, G = N // ROWS_PER_TILE, K // K_PER_TILE
    stream = np.unpackbits(blob.reshape(T, G, THREADS_PER_TILE, 16 * bits),
                           axis=-1, bitorder="little")
    fields = stream.reshape(T, G, THREADS_PER_TILE, ELEMS_PER_THREAD, bits)
    elems = (fields << np.arange(bits, dtype=np.uint8)).sum(axis=-1).astype(np.uint8)
    tiles = np.empty((T, G, ROWS_PER_TILE, K_PER_TILE), dtype=np.uint8)
    tiles[:, :, row, col] = elems
    return np.ascontiguousarray(tiles.transpose(0, 2, 1, 3).reshape(N, K))


def unpack_idxn_scalar(blob: np.ndarray, N: int, K: int, bits: int) -> np.ndarray:
    """Pure-Python restatement of the normative byte/bit addressing
    (idxN.py:37-51), one element at a time — small cases only. Independent of
    the vectorised pair above, used to cross-check it."""
    _check_shape(N, K, bits)
    blob = np.asarray(blob, dtype=np.uint8).reshape(-1)
    out = np.zeros((N, K), dtype=np.uint8)
    tile_bytes = 1024 * bits
    for t in range(N // 128):
        for g in range(K // 64):
            base = (t * (K // 64) + g) * tile_bytes
            for wx in range(2):
                for lane in range(32):
                    chunk = base + wx * 512 * bits + lane * 16 * bits
                    word = int.from_bytes(blob[chunk:chunk + 16 * bits].tobytes(), "little")
                    for p in range(64):
                        kt, v, d, s2 = p // 16, (p // 4) % 4, (p // 2) % 2, p % 2
                        n = t * 128 + wx * 64 + v * 16 + d * 8 + (lane >> 2)
                        k = g * 64 + kt * 16 + 2 * (lane & 3) + 8 * s2
                        pair = (word >> (2 * bits * p)) & ((1 << (2 * bits)) - 1)
                        out[n, k] = pair & ((1 << bits) - 1)
                        out[n, k + 1] = pair >> bits
    return out


# --------------------------------------------------------------------------- #
# dequantisation and the reference forward (src/scripts/palettized_modules.py)
# --------------------------------------------------------------------------- #

def _lut2d(lut: torch.Tensor, bits: int) -> torch.Tensor:
    lut = lut if torch.is_tensor(lut) else torch.from_numpy(np.asarray(lut))
    return lut if lut.dim() == 2 else lut.view(-1, 1 << bits)


def dequant_indices(indices: np.ndarray, lut: torch.Tensor, group_size: int,
                    bits: int) -> torch.Tensor:
    """W[n, k] = float(LUT[min(n // gs, G-1), idx[n, k]]) as fp32 [N, K]
    (palettized_modules.py:149-162: row-group index clamped to the last LUT
    row, LUT cast to fp32 before the gather)."""
    lut = _lut2d(lut, bits)
    N = indices.shape[0]
    rg = (torch.arange(N) // int(group_size)).clamp_(max=lut.shape[0] - 1)
    return lut[rg].float().gather(1, torch.from_numpy(indices.astype(np.int64)))


def dequant(blob, lut: torch.Tensor, N: int, K: int, group_size: int,
            bits: int = 4) -> torch.Tensor:
    """reference_dequant (palettized_modules.py:125-162): blob -> fp32 [N, K]."""
    blob = blob.detach().cpu().numpy() if torch.is_tensor(blob) else blob
    return dequant_indices(unpack_idxn(blob, N, K, bits), lut, group_size, bits)


def dequant_kgrouped(indices: np.ndarray, lut_k: torch.Tensor, group_k: int = 128) -> torch.Tensor:
    """K-grouped palette variant: one 2**b-entry LUT per (K block, output row),
    lut_k [K // group_k, N, 2**b]; W[n, k] = lut_k[k // group_k, n, idx[n, k]].

    The reference has no such mode; it is the composition of reference calls
    with group_size = 1 on each K block (palettized_modules.py:155-156 accepts
    group_size 1), concatenated along K.
    """
    N, K = indices.shape
    cols = []
    for j in range(K // group_k):
        blk = indices[:, j * group_k:(j + 1) * group_k]
        cols.append(dequant_indices(blk, lut_k[j], 1, int(math.log2(lut_k.shape[-1]))))
    return torch.cat(cols, dim=1)


def linear_forward(x: torch.Tensor, w1: torch.Tensor, w2: Optional[torch.Tensor] = None,
                   resA: Optional[torch.Tensor] = None, resB: Optional[torch.Tensor] = None,
                   bias: Optional[torch.Tensor] = None,
                   rot_signs: Optional[torch.Tensor] = None,
                   awq_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """PalettizedLinear.forward, reference branch (palettized_modules.py:1204-1251,
    1360-1369), given already-dequantised fp32 stream weights w1 (and w2).

    x [M, K] or [B, T, K]; rotate first when signs are given (:1235-1236;
    with a scale the compensated form of :624-629); y = x.float() @ w1.T, a
    second stream is a second matmul added in fp32 (:1245-1250); ONE cast to
    x.dtype (:1251); then the low-rank residual in resA's dtype (:1360-1364)
    and the bias (:1365-1366) are added to the already-rounded output.
    """
    shape = x.shape
    if x.dim() == 3:
        x = x.reshape(shape[0] * shape[1], shape[2])
    if rot_signs is not None:
        x = fht_forward_awq(x, rot_signs, awq_scale) if awq_scale is not None \
            else fht_forward(x, rot_signs)
    xf = x.float()
    y = xf @ w1.t()
    if w2 is not None:
        y = y + xf @ w2.t()
    out = y.to(x.dtype)
    if resA is not None and resB is not None:
        xr = x.to(resA.dtype)
        out = out + ((xr @ resB.t()) @ resA.t()).to(out.dtype)
    if bias is not None:
        out = out + bias
    if len(shape) == 3:
        out = out.view(shape[0], shape[1], -1)
    return out


def silu_mul_fused(gate_f32: torch.Tensor, up_f32: torch.Tensor, dtype) -> torch.Tensor:
    """Epilogue of the merged gate+up decode kernel
    (src/flute_extended/src/kernel_gemv_mlp.cu:382-383): on the fp32 sums,
    silu(g) = g / (1 + exp(-g)), times u, rounded ONCE to the output dtype."""
    g = gate_f32.float()
    return (g / (1.0 + torch.exp(-g)) * up_f32.float()).to(dtype)


def mlp_block_unfused(x, wg, wu, wd):
    """down(silu(gate(x)) * up(x)) with three reference modules
    (src/scripts/modeling.py:1001-1003): gate and up outputs are rounded to
    x.dtype before silu*mul, which torch evaluates in that dtype."""
    g = linear_forward(x, wg)
    u = linear_forward(x, wu)
    h = torch.nn.functional.silu(g) * u
    return linear_forward(h, wd)


def mlp_block_fused(x, wg, wu, wd):
    """The decode route of FusedPalettizedMLP (palettized_modules.py:1673-1682):
    fused gate/up epilogue, then down."""
    xf = x.float()
    h = silu_mul_fused(xf @ wg.t(), xf @ wu.t(), x.dtype)
    return linear_forward(h, wd)


# --------------------------------------------------------------------------- #
# Hadamard rotation (src/flute_extended/fht.py)
# --------------------------------------------------------------------------- #

def rotation_signs(K: int, seed: int) -> torch.Tensor:
    """(K,) fp32 +-1 vector, fht.py:105-115: CPU generator seeded seed + 4242,
    randint(0, 2) * 2 - 1. Depends on torch's CPU randint stream; pinned by a
    golden vector in tests/golden/."""
    g = torch.Generator().manual_seed(int(seed) + 4242)
    return torch.randint(0, 2, (int(K),), generator=g).float() * 2 - 1


def fht_segments(K: int) -> List[Tuple[int, int]]:
    """Descending power-of-two split of K as (offset, size), fht.py:118-134."""
    out, off = [], 0
    while off < K:
        b = 1 << ((K - off).bit_length() - 1)
        out.append((off, b))
        off += b
    return out


def _wht(v: torch.Tensor) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard butterfly on the last axis, stage length
    doubling from 1 (fht.py:174-192): in every 2*len group the first half
    becomes a + b and the second a - b. fp32 in, fp32 out."""
    R, n = v.shape
    h = 1
    while h < n:
        w = v.view(R, n // (2 * h), 2, h)
        a, b = w[:, :, 0, :], w[:, :, 1, :]
        v = torch.stack((a + b, a - b), dim=2).reshape(R, n)
        h *= 2
    return v


def fht_forward(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """x @ T: per segment butterfly, then * signs, then * (1/sqrt(b)), fp32
    arithmetic, result in x.dtype (fht.py:206-222)."""
    K = x.shape[-1]
    v = x.reshape(-1, K).float()
    s = signs.float().reshape(1, K)
    out = torch.empty_like(v)
    for off, b in fht_segments(K):
        seg = _wht(v[:, off:off + b].contiguous())
        out[:, off:off + b] = (seg * s[:, off:off + b]) * (1.0 / math.sqrt(b))
    return out.reshape(x.shape).to(x.dtype)


def fht_adjoint(v: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """v @ T^T: signs on the input, butterfly, * (1/sqrt(b)) (fht.py:225-238)."""
    K = v.shape[-1]
    g = v.reshape(-1, K).float()
    s = signs.float().reshape(1, K)
    out = torch.empty_like(g)
    for off, b in fht_segments(K):
        seg = _wht((g[:, off:off + b] * s[:, off:off + b]).contiguous())
        out[:, off:off + b] = seg * (1.0 / math.sqrt(b))
    return out.reshape(v.shape).to(v.dtype)


def embedding_forward(ids: torch.Tensor, idx1: np.ndarray, lut1: torch.Tensor, group_size: int,
                      idx2: Optional[np.ndarray] = None, lut2: Optional[torch.Tensor] = None,
                      resA: Optional[torch.Tensor] = None, resB: Optional[torch.Tensor] = None,
                      rot_signs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ids of a palettized table, the dtype ladder of PalettizedEmbedding.forward
    (src/scripts/palettized_modules.py:2276-2335): per stream
    lut[ids // gs].gather(-1, idx[ids]) in the palette dtype (:2293-2294), the second stream
    added in that dtype with stream 1 first (:2313-2315), widened to fp32, plus
    resA[ids].float() @ resB.float() (:2316-2319), un-rotated through the adjoint transform
    when the table is a tied, rotated head (:2326-2334), one cast to the palette dtype
    (:2335). ids: integer tensor of any shape with values in [0, N); idx*: logical [N, K]
    uint8 codes."""
    ids = ids.long()
    N = idx1.shape[0]
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= N):
        raise ValueError(f"ids out of range [0, {N})")

    def stream(idx, lut):
        assert lut.dim() == 2, "palettes are [n_groups, 2**bits]"
        rows = torch.from_numpy(np.ascontiguousarray(idx))[ids].long()
        return lut[ids // group_size].gather(-1, rows)

    w = stream(idx1, lut1)
    if idx2 is not None:
        w = w + stream(idx2, lut2)
    if resA is not None and resB is not None:
        w = w.float() + (resA[ids].float() @ resB.float())
    else:
        w = w.float()
    if rot_signs is not None:
        w = fht_adjoint(w, rot_signs)
    return w.to(lut1.dtype)


def fht_forward_awq(x: torch.Tensor, signs: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """((x * s) @ T) / s with fp32 multiply, fp32 transform, true fp32 division,
    one cast to x.dtype (fht.py:645-651)."""
    out = fht_forward(x.float() * s.float(), signs).float() / s.float()
    return out.to(x.dtype)


def fht_block(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Normalised Hadamard transform of every `block`-wide slice of the last
    axis, no signs. Composition of the reference's own butterfly:
    fht_reference(x.reshape(-1, block), ones(block)) (fht.py:206-222)."""
    K = x.shape[-1]
    return fht_forward(x.reshape(-1, block), torch.ones(block)).reshape(x.shape)


def hadamard_matrix(n: int) -> torch.Tensor:
    """Sylvester H_n (fht.py:137-148)."""
    H = torch.ones(1, 1)
    while H.shape[0] < n:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return H


def rotation_matrix(signs: torch.Tensor) -> torch.Tensor:
    """Explicit block-diagonal T for a sign vector (fht.py:151-167)."""
    K = signs.numel()
    T = torch.zeros(K, K)
    for off, b in fht_segments(K):
        T[off:off + b, off:off + b] = hadamard_matrix(b) * signs[off:off + b].view(1, b) / math.sqrt(b)
    return T


# --------------------------------------------------------------------------- #
# error measures used by the parity tests
# --------------------------------------------------------------------------- #

def max_rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want| — the relative-error form of the
    reference's own gate (src/flute_extended/test_qwen_weights.py:96-121)."""
    g, w = got.double(), want.double()
    return float((g - w).abs().max() / w.abs().max().clamp_min(1e-30))


def cosine(got: torch.Tensor, want: torch.Tensor) -> float:
    """Cosine similarity of the flattened tensors
    (src/flute_extended/benchmark_kernel.py:95-107)."""
    g, w = got.double().flatten(), want.double().flatten()
    return float((g @ w) / (g.norm() * w.norm()).clamp_min(1e-30))
