"""CPU-side checks: the C-ABI library loads and exports every symbol the header
declares, argument validation answers without touching a GPU, the host idxN tool
matches the reference-made golden blobs, and the Python surface mirrors the
reference's constructor contracts."""
from __future__ import annotations

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, load_pkg

pkg = load_pkg()
HEADER = os.path.join(ROOT, "include", "b200_lut.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200lut_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = pkg._lib.lib()
    names = _declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(L, name), f"{name} declared in include/b200_lut.h but not exported"
    assert set(names) == set(pkg._lib.EXPORTS)
    assert L.b200lut_version() >= 100


def test_packed_bytes_and_shape_refusals():
    L = pkg._lib.lib()
    assert L.b200lut_packed_bytes(4096, 4096, 4) == 4096 * 4096 // 2
    assert L.b200lut_packed_bytes(12288, 4096, 3) == 12288 * 4096 * 3 // 8
    assert L.b200lut_packed_bytes(100, 64, 4) == 0
    assert L.b200lut_packed_bytes(128, 60, 4) == 0
    assert L.b200lut_packed_bytes(128, 64, 5) == 0
    with pytest.raises(ValueError):
        pkg._lib.packed_bytes(128, 64, 0)


def test_validation_errors_carry_a_message():
    L = pkg._lib.lib()
    rc = L.b200lut_repack_from_idxn(None, None, 100, 64, 4, None)
    assert rc == 1 and b"multiple of 128" in L.b200lut_last_error()
    rc = L.b200lut_gemv(None, None, None, None, 1, 128, 64, 4, 128, 1, 0, 0, None, 0, None)
    assert rc == 1 and b"null" in L.b200lut_last_error()
    buf = ctypes.create_string_buffer(64)
    seg = pkg._lib.Segment()
    seg.packed = seg.lut = seg.out = ctypes.addressof(buf) & ~15
    seg.N, seg.group_size, seg.n_groups, seg.bits, seg.ldo = 128, 128, 1, 4, 128
    x = ctypes.addressof(buf) & ~15
    rc = L.b200lut_gemv_multi(x, 64, 17, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, None)
    assert rc == 2 and b"M <= 16" in L.b200lut_last_error() or b"16" in L.b200lut_last_error()
    seg.group_size = 48
    rc = L.b200lut_gemv_multi(x, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, None)
    assert rc == 2 and b"group_size" in L.b200lut_last_error()
    seg.group_size, seg.res_rank = 128, 12
    rc = L.b200lut_gemv_multi(x, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, None)
    assert rc == 2 and b"residual rank" in L.b200lut_last_error()
    seg.res_rank = 16
    rc = L.b200lut_gemv_multi(x, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, None)
    assert rc == 1 and b"resA" in L.b200lut_last_error()
    rc = L.b200lut_gemm(x, 64, 32, 64, 0, ctypes.byref(seg), 0, 0, None)
    assert rc == 1 and b"b200lut_residual_project_rows" in L.b200lut_last_error()
    seg.res_rank = 12                                   # the prefill GEMM wants a multiple of 8 too
    rc = L.b200lut_gemm(x, 64, 32, 64, 0, ctypes.byref(seg), 0, 0, None)
    assert rc == 2 and b"multiple of 8" in L.b200lut_last_error()
    rc = L.b200lut_residual_project_rows(x, 64, 32, 64, 0, x, 8, x, 64, 32, 0, None)
    assert rc == 1 and b"multiple of 64" in L.b200lut_last_error()
    seg.res_rank = 0
    # the split schedule's workspace: sized without a device (148 SMs assumed), validated like
    # the plain entry
    assert L.b200lut_gemm_workspace_bytes(2048, 4096, 4096) == 0   # 108 tiles left over: no SM to spare
    assert L.b200lut_gemm_workspace_bytes(16, 64, 4096) == 0
    assert L.b200lut_gemm_workspace_bytes(512, 12288, 4096) == 4096 + 44 * 3 * 256 * 128 * 4
    rc = L.b200lut_gemm_ws(x, 64, 32, 60, 0, ctypes.byref(seg), 0, 0, x, 1 << 20, None)
    assert rc == 1 and b"multiple of 64" in L.b200lut_last_error()
    rc = L.b200lut_residual_project(x, 64, 17, 64, 0, x, 8, x, 8, 0, None)
    assert rc == 2 and b"M=17" in L.b200lut_last_error()
    rc = L.b200lut_residual_project(x, 64, 1, 64, 0, None, 8, x, 8, 0, None)
    assert rc == 1 and b"null" in L.b200lut_last_error()
    inp = pkg._lib.Input()
    inp.per_segment, inp.rot_signs = 1, x                   # a launch-wide fold next to per-segment ones
    rc = L.b200lut_gemv_input(x, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, None, ctypes.byref(inp), None)
    assert rc == 1 and b"per-segment folds" in L.b200lut_last_error()
    inp.rot_signs = None
    inp.seg_awq_scale[0] = x                                 # a scale without signs
    rc = L.b200lut_gemv_input(x, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, None, ctypes.byref(inp), None)
    assert rc == 1 and b"segment 0" in L.b200lut_last_error()
    # K-grouped tensor-core form: one palette per 128 input columns
    L.b200lut_gemm_kgrouped.restype = ctypes.c_int
    rc = L.b200lut_gemm_kgrouped(x, 64, 32, 64, 0, x, x, None, 128, 4, x, 128, 0, None, 0, None)
    assert rc == 1 and b"multiple of 128" in L.b200lut_last_error()
    rc = L.b200lut_gemm_kgrouped(x, 128, 32, 128, 0, x, x, None, 128, 5, x, 128, 0, None, 0, None)
    assert rc == 1 and b"code width" in L.b200lut_last_error()
    rc = L.b200lut_gemm_kgrouped(x, 128, 32, 128, 0, x, None, None, 128, 4, x, 128, 0, None, 0, None)
    assert rc == 1 and b"null" in L.b200lut_last_error()
    # an exchange's wait bound is 0 (default) or 1..1000 ms
    ex = pkg._lib.Exchange()
    ex.world, ex.rank, ex.wait, ex.producer_blocks, ex.wait_ms = 2, 0, 1, 4, 5000
    ex.flags = ex.wait_ticket = ex.wait_count = x
    rc = L.b200lut_gemv_exchange(x, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0, ctypes.byref(ex), None)
    assert rc == 1 and b"wait_ms" in L.b200lut_last_error()
    rc = L.b200lut_gemm_multi(x, 64, 32, 128, 0, ctypes.byref(seg), 5, 0, None, 0, None)
    assert rc == 2 and b"nseg" in L.b200lut_last_error()
    rc = L.b200lut_gemm_multi(x, 64, 32, 64, 0, ctypes.byref(seg), 1, 0, None, 0, None)
    assert rc == 1 and b"at least 128" in L.b200lut_last_error()
    rc = L.b200lut_gemv_kgrouped(x, 128, 17, 128, 0, x, x, None, 128, 4, x, 128, 1, None, 0, None)
    assert rc == 2 and b"M=17" in L.b200lut_last_error()
    rc = L.b200lut_gemv_kgrouped(x, 128, 1, 192, 0, x, x, None, 128, 4, x, 128, 1, None, 0, None)
    assert rc == 1 and b"multiples of 128" in L.b200lut_last_error()
    rc = L.b200lut_gemv_kgrouped(x, 256, 1, 256, 0, x, x, None, 128, 4, x, 128, 2, None, 0, None)
    assert rc == 4 and b"workspace" in L.b200lut_last_error()
    assert L.b200lut_gemv_kgrouped_workspace_bytes(256, 4, 1) == 0
    assert L.b200lut_gemv_kgrouped_workspace_bytes(256, 4, 3) == 2 * 4 + 256 + 3 * 4 * 256 * 4
    rc = L.b200lut_gemm_two_stream(x, 128, 32, 128, 0, ctypes.byref(seg), 0, x, 1 << 20, None)
    assert rc == 1 and b"second stream" in L.b200lut_last_error()
    assert L.b200lut_gemm_two_stream_bytes(32, 128) == 32 * 128 * 4
    rc = L.b200lut_embed_gather(x, 4, 60, 0, ctypes.byref(seg), None, 0, None)
    assert rc == 1 and b"K %% 64" in L.b200lut_last_error() or b"64" in L.b200lut_last_error()
    rc = L.b200lut_embed_gather(x, -1, 64, 0, ctypes.byref(seg), None, 0, None)
    assert rc == 1 and b"n_ids" in L.b200lut_last_error()
    seg.res_rank = 4
    rc = L.b200lut_embed_gather(x, 4, 64, 0, ctypes.byref(seg), None, 0, None)
    assert rc == 1 and b"resA and resB" in L.b200lut_last_error()
    seg.res_rank = 0
    assert L.b200lut_embed_gather(None, 0, 64, 0, ctypes.byref(seg), None, 0, None) == 0   # no ids: no launch
    rc = L.b200lut_round_rows(None, 8, None, 4, 2, 8, 0, None)
    assert rc == 1 and b"strides" in L.b200lut_last_error()
    rc = L.b200lut_silu_mul(x, x, 4, 12, 16, 16, 0, None)
    assert rc == 1 and b"multiple of 8" in L.b200lut_last_error()
    rc = L.b200lut_silu_mul(x, x, 4, 16, 12, 16, 0, None)
    assert rc == 5 and b"aligned" in L.b200lut_last_error()
    rc = L.b200lut_fht(x, x, None, None, 1, 96, 96, 96, 0, 0, 64, None)
    assert rc == 1 and b"block" in L.b200lut_last_error()


def test_exchange_descriptor_is_validated_before_any_launch():
    L = pkg._lib.lib()
    buf = ctypes.create_string_buffer(256)
    a = (ctypes.addressof(buf) + 15) & ~15
    seg = pkg._lib.Segment()
    seg.packed = seg.lut = seg.out = a
    seg.N, seg.group_size, seg.n_groups, seg.bits, seg.ldo = 128, 128, 1, 4, 128
    ex = pkg._lib.Exchange()
    ex.world, ex.rank, ex.push, ex.producer_blocks = 9, 0, 1, 1
    call = lambda: L.b200lut_gemv_exchange(a, 64, 1, 64, 0, ctypes.byref(seg), 1, 0, 0, None, 0, 0,
                                           ctypes.byref(ex), None)
    assert call() == 1 and b"world" in L.b200lut_last_error()
    ex.world, ex.rank = 2, 2
    assert call() == 1 and b"rank" in L.b200lut_last_error()
    ex.rank, ex.producer_blocks = 1, 0
    assert call() == 1 and b"producer_blocks" in L.b200lut_last_error()
    ex.producer_blocks = 3
    assert call() == 1 and b"ticket and count" in L.b200lut_last_error()
    ex.ticket, ex.epoch = a + 64, a + 96
    assert call() == 1 and b"flag of rank 0" in L.b200lut_last_error()
    ex.push, ex.wait = 0, 1
    assert call() == 1 and b"flag array" in L.b200lut_last_error()
    ex.flags = a
    assert call() == 1 and b"wait needs its ticket" in L.b200lut_last_error()
    assert L.b200lut_peer_export(None, None, None) == 1
    assert L.b200lut_peer_open(None, None) == 1
    assert L.b200lut_peer_close(None) == 1


def test_workspace_query():
    L = pkg._lib.lib()
    assert L.b200lut_gemv_workspace_bytes(4096, 1, 8) == 0        # cluster fold: no scratch
    n = L.b200lut_gemv_workspace_bytes(4096, 1, 16)
    assert n == 16 * 32 * 2 * 1 * 128 * 4 + 32 * 4


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
def test_host_idxn_matches_reference_blobs(golden, bits):
    for (N, K) in ((128, 64), (256, 128)):
        tag = f"idxn_b{bits}_{N}x{K}"
        idx, blob = golden.np(tag + "_idx"), golden.np(tag + "_blob")
        assert np.array_equal(pkg.idxN.pack_idxn(idx, bits), blob)
        assert np.array_equal(pkg.idxN.unpack_idxn(blob, N, K, bits), idx)


def test_host_idxn_self_test_and_refusals():
    assert pkg.idxN.self_test()
    with pytest.raises(ValueError):
        pkg.idxN.pack_idxn(np.zeros((64, 64), np.uint8), 4)
    with pytest.raises(ValueError):
        pkg.idxN.pack_idxn(np.full((128, 64), 4, np.uint8), 2)
    with pytest.raises(ValueError):
        pkg.idxN.unpack_idxn(np.zeros(100, np.uint8), 128, 64, 4)
    rows = np.random.default_rng(1).integers(0, 256, size=(128, 24), dtype=np.uint8)
    blob = pkg.idxN.pack_idxn_from_packed(rows, 3)
    idx = pkg.idxN.unpack_idxn(blob, 128, 64, 3)
    assert np.array_equal(np.packbits(((idx[:, :, None] >> np.arange(3)) & 1).reshape(128, -1),
                                      axis=1, bitorder="little"), rows)


def test_signs_and_segments_match_golden(golden):
    for (K, seed) in ((64, 0), (1024, 7), (4096, 0), (12288, 3)):
        s = pkg.fht.rotation_signs(K, seed)
        assert np.array_equal(s.to(torch.int8).numpy(), golden.np(f"signs_K{K}_s{seed}"))
    assert pkg.fht.segments(12288) == [(0, 8192), (8192, 4096)]
    assert pkg.fht.segments(3072) == [(0, 2048), (2048, 1024)]
    T = pkg.fht.build_rotation_matrix(64, 0)
    assert torch.allclose(T @ T.t(), torch.eye(64), atol=1e-6)


def test_constructor_contracts():
    PL = pkg.PalettizedLinear
    blob = torch.zeros(128 * 64 // 2, dtype=torch.uint8)
    lut = torch.zeros(1, 16, dtype=torch.bfloat16)
    m = PL(blob, lut, 4, 128, 128, 64)
    assert (m.N, m.K, m.bitwidth, m.group_size, m.bitwidth2) == (128, 64, 4, 128, 4)
    assert not m.has_stream2 and not m.has_residual() and m.rot_signs is None
    with pytest.raises(ValueError, match="N%128"):
        PL(blob, lut, 4, 128, 100, 64)
    with pytest.raises(ValueError, match="blob numel"):
        PL(blob[:-1], lut, 4, 128, 128, 64)
    with pytest.raises(ValueError, match="BOTH"):
        PL(blob, lut, 4, 128, 128, 64, indices2=blob)
    with pytest.raises(ValueError, match="rotation_k"):
        PL(blob, lut, 4, 128, 128, 64, rotation_seed=1, rotation_k=128)
    with pytest.raises(ValueError, match="without rotation"):
        PL(blob, lut, 4, 128, 128, 64, awq_scale=torch.ones(64))
    with pytest.raises(ValueError, match="finite and positive"):
        PL(blob, lut, 4, 128, 128, 64, rotation_seed=1, rotation_k=64, awq_scale=torch.zeros(64))
    r = PL(blob, lut, 4, 128, 128, 64, rotation_seed=3, rotation_k=64, awq_scale=torch.ones(64))
    assert r.fold_order == "rotate_then_awq"
    assert torch.equal(r.rot_signs, pkg.fht.rotation_signs(64, 3))
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 64, dtype=torch.bfloat16))       # no CPU compute route
    codes = np.random.default_rng(0).integers(0, 16, size=(128, 64), dtype=np.uint8)
    m2 = PL(torch.from_numpy(pkg.idxN.pack_idxn(codes, 4)), lut, 4, 128, 128, 64)
    assert np.array_equal(m2._logical_indices_numpy(), codes)


def test_plan_entries_refuse_null_buffers_before_any_cuda_call():
    L = pkg._lib
    lib = L.lib()
    assert lib.b200lut_plan_form(None) < 0                      # not a plan buffer
    assert lib.b200lut_plan_release(None) == 0                  # nothing to drop
    assert lib.b200lut_plan_status(None) == L.ERR_INVALID if hasattr(L, "ERR_INVALID") else lib.b200lut_plan_status(None) != 0
    assert lib.b200lut_plan_run(None, 1, L.dtype_id(torch.bfloat16), None) != 0
    assert lib.b200lut_plan_bytes(None, 0, 1, L.dtype_id(torch.bfloat16)) == 0


def test_missing_library_is_loud(monkeypatch):
    monkeypatch.setattr(pkg._lib, "_lib", None)
    monkeypatch.setattr(pkg._lib, "LIB_PATH", "/nonexistent/libb200lut.so")
    with pytest.raises(RuntimeError, match="missing"):
        pkg._lib.lib()
