"""Host-side producer / verifier of the idxN packed-index blobs (idx1..idx4).

Mirrors the interface of the reference's format module
(src/flute_extended/flute_extended/idxN.py: pack_idxn :235, unpack_idxn :267,
blob_bytes :111, check_eligible :103, pack_idxn_from_packed :294, self_test :311)
so artifact tooling written against it keeps working. This is the on-disk
format tool (numpy, host); the GPU consumes blobs through
b200lut_repack_from_idxn, which converts them once into the library's own slab
layout.

Blob layout (normative, idxN.py:37-55 of the reference): one tile of 1024*bits
bytes per (128-row tile t, 64-k tile g) at ((t * K/64) + g) * 1024*bits; in a
tile, thread chunk th = wx*32 + lane (16*bits bytes) holds 128 fields of `bits`
bits, LSB-first; field e = 2*p + j, p = kt*16 + v*4 + d*2 + s2, is the code of
row wx*64 + v*16 + d*8 + (lane >> 2), k = kt*16 + 2*(lane & 3) + 8*s2 + j.
"""
from __future__ import annotations

import functools

import numpy as np

ROWS_PER_TILE = 128
K_PER_GROUP = 64
PAIRS_PER_CHUNK = 64
TILE_THREADS = 64
TILE_BYTES_PER_BIT = 1024
BITS_SUPPORTED = (1, 2, 3, 4)
_TILE_ELEMS = ROWS_PER_TILE * K_PER_GROUP


def check_bits(bits: int) -> int:
    b = int(bits)
    if b not in BITS_SUPPORTED:
        raise ValueError(f"idxN supports bit widths {BITS_SUPPORTED}, got bits={bits}")
    return b


def check_eligible(N: int, K: int) -> None:
    if N % ROWS_PER_TILE != 0:
        raise ValueError(f"idxN layout requires N % 128 == 0, got N={N}")
    if K % K_PER_GROUP != 0:
        raise ValueError(f"idxN layout requires K % 64 == 0, got K={K}")


def blob_bytes(N: int, K: int, bits: int) -> int:
    check_bits(bits)
    return (int(N) * int(K) * int(bits)) // 8


def packed_row_bytes(K: int, bits: int) -> int:
    check_bits(bits)
    return (int(K) * int(bits)) // 8


@functools.lru_cache(maxsize=1)
def _tile_permutation() -> np.ndarray:
    """perm[q] = tile-local flat index (row * 64 + k) of the q-th field of a tile
    in blob order (q = th * 128 + e). Width-independent."""
    q = np.arange(_TILE_ELEMS)
    th, e = q >> 7, q & 127
    wx, lane = th >> 5, th & 31
    j, p = e & 1, e >> 1
    s2, d, v, kt = p & 1, (p >> 1) & 1, (p >> 2) & 3, p >> 4
    row = wx * 64 + v * 16 + d * 8 + (lane >> 2)
    col = kt * 16 + 2 * (lane & 3) + 8 * s2 + j
    perm = row * K_PER_GROUP + col
    assert np.array_equal(np.sort(perm), q)
    return perm


def pack_idxn(indices: np.ndarray, bits: int) -> np.ndarray:
    """Logical codes [N, K] (values < 2**bits) -> idxN blob (uint8, 1-D)."""
    b = check_bits(bits)
    idx = np.ascontiguousarray(indices, dtype=np.uint8)
    if idx.ndim != 2:
        raise ValueError(f"expected a 2-D index matrix, got shape {idx.shape}")
    N, K = idx.shape
    check_eligible(N, K)
    if idx.size and int(idx.max()) >= (1 << b):
        raise ValueError(f"idx{b} indices must be < {1 << b}, got max {int(idx.max())}")
    T, G = N // ROWS_PER_TILE, K // K_PER_GROUP
    tiles = idx.reshape(T, ROWS_PER_TILE, G, K_PER_GROUP).swapaxes(1, 2).reshape(T * G, _TILE_ELEMS)
    fields = tiles[:, _tile_permutation()]
    if b == 4:      # two fields per byte: the common case, no bit explosion
        return np.ascontiguousarray(fields[:, 0::2] | (fields[:, 1::2] << 4)).reshape(-1)
    bitplanes = (fields[:, :, None] >> np.arange(b, dtype=np.uint8)) & 1
    return np.packbits(bitplanes.reshape(T * G, _TILE_ELEMS * b), axis=1, bitorder="little").reshape(-1)


def unpack_idxn(blob: np.ndarray, N: int, K: int, bits: int) -> np.ndarray:
    """idxN blob -> logical codes [N, K] uint8."""
    b = check_bits(bits)
    check_eligible(N, K)
    blob = np.ascontiguousarray(blob, dtype=np.uint8).reshape(-1)
    expected = blob_bytes(N, K, b)
    if blob.size != expected:
        raise ValueError(f"idx{b} blob has {blob.size} bytes, expected N*K*{b}/8 = {expected} "
                         f"(N={N}, K={K})")
    T, G = N // ROWS_PER_TILE, K // K_PER_GROUP
    raw = blob.reshape(T * G, TILE_BYTES_PER_BIT * b)
    if b == 4:
        fields = np.empty((T * G, _TILE_ELEMS), dtype=np.uint8)
        fields[:, 0::2] = raw & 0x0F
        fields[:, 1::2] = raw >> 4
    else:
        bitstream = np.unpackbits(raw, axis=1, bitorder="little").reshape(T * G, _TILE_ELEMS, b)
        fields = np.zeros((T * G, _TILE_ELEMS), dtype=np.uint8)
        for i in range(b):
            fields |= bitstream[:, :, i] << i
    tiles = np.empty_like(fields)
    tiles[:, _tile_permutation()] = fields
    return np.ascontiguousarray(
        tiles.reshape(T, G, ROWS_PER_TILE, K_PER_GROUP).swapaxes(1, 2).reshape(N, K))


def pack_idxn_from_packed(q: np.ndarray, bits: int) -> np.ndarray:
    """Row-major LSB-first packed stream [N, K*bits/8] -> idxN blob."""
    b = check_bits(bits)
    q = np.ascontiguousarray(q, dtype=np.uint8)
    if q.ndim != 2:
        raise ValueError(f"expected a 2-D packed matrix, got shape {q.shape}")
    N = q.shape[0]
    K = (q.shape[1] * 8) // b
    stream = np.unpackbits(q, axis=1, bitorder="little").reshape(N, K, b)
    idx = np.zeros((N, K), dtype=np.uint8)
    for i in range(b):
        idx |= stream[:, :, i] << i
    return pack_idxn(idx, b)


def self_test(shapes=((128, 64), (256, 128), (384, 192), (1024, 512)),
              bits_all=BITS_SUPPORTED) -> bool:
    """pack -> unpack round trip at every width; a blob read at the wrong width
    must be refused."""
    rng = np.random.default_rng(0)
    for b in bits_all:
        for N, K in shapes:
            idx = rng.integers(0, 1 << b, size=(N, K), dtype=np.uint8)
            blob = pack_idxn(idx, b)
            assert blob.size == blob_bytes(N, K, b)
            assert np.array_equal(unpack_idxn(blob, N, K, b), idx), (b, N, K)
            try:
                unpack_idxn(blob, N, K, 4 if b != 4 else 2)
            except ValueError:
                pass
            else:
                raise AssertionError("width confusion not caught")
    return True
