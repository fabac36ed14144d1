"""GPU parity of the embedding gather (b200lut_embed_gather behind PalettizedEmbedding).

Against tests/golden/embedding_vectors.npz (outputs of the reference's own
PalettizedEmbedding.forward) and against the CPU oracle on seeded tables. A gather is
integer work plus one or two palette reads: results are BIT-EXACT wherever no fp32 sum
is involved (one or two streams, and the un-rotation, whose butterfly order is the
reference's); with a low-rank residual the fp32 rank sum runs in ascending order here and
in the reference's matmul order there: max |got - want| / max |want| <= 2^-9 (one 16-bit
rounding of the output)."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from helpers import pkg, rel_err
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib
RES_TOL = 2.0 ** -9


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0


def _golden_module(g, name):
    N, K, gs, bits, bits2, rank, rot = (int(v) for v in g.np(name + "_meta"))
    kw = {}
    if bits2:
        kw.update(indices2=torch.from_numpy(orc.pack_idxn(g.np(name + "_codes2"), bits2)),
                  lut2=g.t(name + "_lut2"), bitwidth2=bits2)
    if rank:
        kw.update(resA=g.t(name + "_resA"), resB=g.t(name + "_resB"))
    if rot >= 0:
        kw.update(rotation_seed=rot, rotation_k=K)
    blob = torch.from_numpy(orc.pack_idxn(g.np(name + "_codes"), bits))
    return pkg.PalettizedEmbedding(blob, g.t(name + "_lut"), bits, gs, N, K, **kw).cuda(), rank


@pytest.mark.parametrize("name", ("e1", "e2", "e3", "e4", "e5", "e6", "e7"))
def test_reference_vectors(golden_embedding, name):
    g = golden_embedding
    mod, rank = _golden_module(g, name)
    want = g.t(name + "_out")
    got = mod(g.t(name + "_ids").cuda()).cpu()
    assert got.shape == want.shape and got.dtype == want.dtype
    if rank:
        assert rel_err(got, want) <= RES_TOL
    else:
        assert torch.equal(got, want)
    # ids on the host, and 32-bit ids, give the same rows
    assert torch.equal(mod(g.t(name + "_ids")).cpu(), got)
    assert torch.equal(mod(g.t(name + "_ids").int().cuda()).cpu(), got)


@pytest.mark.parametrize("N,K,gs,bits,bits2,rank,rot,dtype,n_ids", (
    (2048, 4096, 128, 4, None, 0, None, torch.bfloat16, (4, 250)),   # the 9B hidden size
    (1024, 1024, 64, 3, 2, 0, None, torch.float16, (777,)),
    (512, 12288, 128, 4, None, 0, 17, torch.bfloat16, (33,)),        # 8192 + 4096 segments
    (384, 320, 32, 2, 1, 0, None, torch.bfloat16, (1,)),
    (1280, 2048, 256, 4, 4, 32, None, torch.float16, (65,)),         # deployed recipe: rank 32
    (256, 512, 128, 1, None, 8, 4, torch.bfloat16, (19,)),
    (640, 192, 32, 4, None, 0, None, torch.float16, (300,)),         # fewer (chunk, lane) items than threads
    (1024, 8192, 512, 4, None, 0, None, torch.bfloat16, (3, 7)),     # two items per thread, a group of four tiles
))
def test_seeded_tables_against_the_oracle(N, K, gs, bits, bits2, rank, rot, dtype, n_ids):
    rng = np.random.default_rng(N + K)
    g = torch.Generator().manual_seed(N + K)
    ng = -(-N // gs)
    codes = rng.integers(0, 1 << bits, size=(N, K), dtype=np.uint8)
    lut = (0.02 * torch.randn(ng, 1 << bits, generator=g)).to(dtype)
    kw, okw = {}, {}
    if bits2:
        codes2 = rng.integers(0, 1 << bits2, size=(N, K), dtype=np.uint8)
        lut2 = (0.005 * torch.randn(ng, 1 << bits2, generator=g)).to(dtype)
        kw.update(indices2=torch.from_numpy(orc.pack_idxn(codes2, bits2)), lut2=lut2, bitwidth2=bits2)
        okw.update(idx2=codes2, lut2=lut2)
    if rank:
        resA = (0.05 * torch.randn(N, rank, generator=g)).to(dtype)
        resB = (0.05 * torch.randn(rank, K, generator=g)).to(dtype)
        kw.update(resA=resA, resB=resB)
        okw.update(resA=resA, resB=resB)
    if rot is not None:
        kw.update(rotation_seed=rot, rotation_k=K)
        okw.update(rot_signs=orc.rotation_signs(K, rot))
    mod = pkg.PalettizedEmbedding(torch.from_numpy(orc.pack_idxn(codes, bits)), lut, bits, gs, N, K,
                                  **kw).cuda()
    ids = torch.from_numpy(rng.integers(0, N, size=n_ids, dtype=np.int64))
    ids.view(-1)[0] = N - 1
    got = mod(ids.cuda()).cpu()
    want = orc.embedding_forward(ids, codes, lut, gs, **okw)
    assert got.shape == tuple(n_ids) + (K,) and got.dtype == dtype
    if rank:
        assert rel_err(got, want) <= RES_TOL
    else:
        assert torch.equal(got, want)


def test_empty_ids_and_repeated_ids():
    codes = np.random.default_rng(1).integers(0, 16, size=(128, 64), dtype=np.uint8)
    lut = (0.02 * torch.randn(1, 16, generator=torch.Generator().manual_seed(1))).half()
    mod = pkg.PalettizedEmbedding(torch.from_numpy(orc.pack_idxn(codes, 4)), lut, 4, 128, 128, 64).cuda()
    out = mod(torch.empty(0, 3, dtype=torch.int64, device="cuda"))
    assert out.shape == (0, 3, 64) and out.dtype == torch.float16
    ids = torch.tensor([5, 5, 127, 5])
    got = mod(ids.cuda()).cpu()
    assert torch.equal(got, orc.embedding_forward(ids, codes, lut, 128))
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[3])


def test_an_id_outside_the_table_gives_zeros_and_a_status_not_a_fault():
    codes = np.random.default_rng(2).integers(0, 16, size=(256, 128), dtype=np.uint8)
    lut = (0.02 * torch.randn(2, 16, generator=torch.Generator().manual_seed(2))).to(torch.bfloat16)
    mod = pkg.PalettizedEmbedding(torch.from_numpy(orc.pack_idxn(codes, 4)), lut, 4, 128, 256, 128).cuda()
    ids = torch.tensor([3, 256, -1, 255])
    got = mod(ids.cuda()).cpu()
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0x6000
    assert L.lib().b200lut_device_status() == 0          # reading clears the word
    good = orc.embedding_forward(torch.tensor([3, 255]), codes, lut, 128)
    assert torch.equal(got[0], good[0]) and torch.equal(got[3], good[1])
    assert not got[1].any() and not got[2].any()
    with pytest.raises(ValueError, match="out of range"):
        mod(ids)                                          # host ids are checked on the host


def test_c_entry_with_a_strided_unaligned_output():
    N, K = 256, 192
    codes = np.random.default_rng(3).integers(0, 8, size=(N, K), dtype=np.uint8)
    lut = (0.02 * torch.randn(2, 8, generator=torch.Generator().manual_seed(3))).half()
    packed = L.repack_from_idxn(torch.from_numpy(orc.pack_idxn(codes, 3)).cuda(), N, K, 3)
    ids = torch.tensor([0, 200, 17, 255, 128], device="cuda")
    buf = torch.full((5, K + 10), 3.0, dtype=torch.float16, device="cuda")
    seg = (L.Segment * 1)()
    s = seg[0]
    lut_d = lut.cuda()
    s.packed, s.lut, s.bits = packed.data_ptr(), lut_d.data_ptr(), 3
    s.N, s.group_size, s.n_groups = N, 128, 2
    s.out, s.ldo = buf.data_ptr() + 2 * 3, K + 10          # 6 bytes off the 16-byte grid
    L.check(L.lib().b200lut_embed_gather(ids.data_ptr(), 5, K, L.dtype_id(torch.float16), seg, None, 0,
                                         L._stream(ids)))
    want = orc.embedding_forward(ids.cpu(), codes, lut, 128)
    assert torch.equal(buf[:, 3:3 + K].cpu(), want)
    assert (buf[:, :3] == 3.0).all() and (buf[:, 3 + K:] == 3.0).all()
    # fp32 rows, then the library's own rounding pass
    s.out, s.ldo = 0, K
    w = torch.empty(5, K, dtype=torch.float32, device="cuda")
    s.out = w.data_ptr()
    L.check(L.lib().b200lut_embed_gather(ids.data_ptr(), 5, K, L.dtype_id(torch.float16), seg, None, 1,
                                         L._stream(ids)))
    assert torch.equal(w.cpu(), want.float())
    assert torch.equal(L.round_rows(w, torch.float16).cpu(), want)


def test_cuda_ids_out_of_range_are_zero_rows_and_reported():
    """Ids that live on the device cannot be refused before the launch without a host sync: the
    kernel writes zero rows for them (the reference asserts on the device and loses the context,
    src/scripts/palettized_modules.py:1957-1976, 2300-2306); the module records it and check_ids()
    raises. Ids on the host are refused up front, as the reference does."""
    N, K = 256, 128
    codes, blob = pkg.synthetic.make_blob(N, K, 4, 5)
    lut = pkg.synthetic.make_lut(N // 128, 4, torch.bfloat16, 5)
    emb = pkg.PalettizedEmbedding(blob, lut, 4, 128, N, K).cuda()
    good = torch.tensor([0, 5, 255], device="cuda")
    emb(good)
    emb.check_ids()                                   # nothing recorded
    rows = emb(torch.tensor([3, N, -1, 7], device="cuda"))
    assert bool((rows[1] == 0).all()) and bool((rows[2] == 0).all())
    assert torch.equal(rows[0], emb(torch.tensor([3], device="cuda"))[0])
    with pytest.raises(ValueError, match="out of range"):
        emb.check_ids()
    emb.check_ids()                                   # the record is cleared
    assert pkg._lib.lib().b200lut_device_status() == 0
    with pytest.raises(ValueError, match="out of range"):
        emb(torch.tensor([N]))
