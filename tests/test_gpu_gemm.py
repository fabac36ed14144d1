"""GPU parity of the prefill GEMM (M > 16, tcgen05 / TMEM) against the CPU oracle.

Tolerance: max |got - want| / max |want| <= 1e-2 (16-bit output, fp32 accumulate).
Dequantised weights are checked BIT-EXACT through the same kernel with one-hot
activations (1.0 * w + zeros is exact in fp32 and in the 16-bit output)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOL, Case, pkg, rel_err
from oracle import lut_linear_oracle as orc

pytestmark = pytest.mark.gpu
L = pkg._lib


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    torch.cuda.synchronize()
    assert L.lib().b200lut_device_status() == 0, "a bounded wait ran out inside a kernel"


@pytest.mark.parametrize("N,K,gs,dtype,M", (
    (128, 64, 128, torch.bfloat16, 17),
    (256, 256, 128, torch.bfloat16, 32),
    (512, 1024, 64, torch.float16, 100),
    (1024, 4096, 128, torch.bfloat16, 128),
    (384, 512, 32, torch.bfloat16, 64),
    (1024, 1024, 128, torch.float16, 300),
    (256, 2048, 128, torch.bfloat16, 513),
))
def test_gemm_matches_oracle(N, K, gs, dtype, M):
    case = Case(N, K, gs, 4, dtype, seed=N + K + M)
    x = case.x(M)
    got = case.module()(x.cuda())
    assert got.shape == (M, N) and not torch.isnan(got.float()).any()
    assert rel_err(got, case.oracle(x)) <= TOL


@pytest.mark.parametrize("gs,dtype", ((128, torch.bfloat16), (64, torch.float16), (32, torch.bfloat16)))
def test_weights_through_the_gemm_are_bit_exact(gs, dtype):
    N, K = 256, 192
    case = Case(N, K, gs, 4, dtype, seed=gs)
    x = torch.zeros(K, K, dtype=dtype)
    x[torch.arange(K), torch.arange(K)] = 1.0
    W = case.module()(x.cuda()).cpu().t()          # [N, K]
    assert torch.equal(W.float(), case.w1)


@pytest.mark.parametrize("bits,gs,dtype,N,K,M", (
    (3, 128, torch.bfloat16, 512, 1024, 128),      # hybrid recipe: 3-bit codes, 8-entry palettes
    (3, 64, torch.float16, 256, 192, 40),
    (2, 128, torch.bfloat16, 256, 512, 257),
    (1, 64, torch.bfloat16, 128, 128, 33),
))
def test_sub_4_bit_widths_on_the_tensor_core_gemm(bits, gs, dtype, N, K, M):
    case = Case(N, K, gs, bits, dtype, seed=bits * 100 + gs, bias=True)
    x = case.x(M)
    assert rel_err(case.module()(x.cuda()), case.oracle(x)) <= TOL
    # and the dequantised weights come through bit-exact
    eye = torch.zeros(K, K, dtype=dtype)
    eye[torch.arange(K), torch.arange(K)] = 1.0
    plain = Case(N, K, gs, bits, dtype, seed=bits * 100 + gs)
    W = plain.module()(eye.cuda()).cpu().t()
    assert torch.equal(W.float(), plain.w1)


def test_bias_second_stream_and_token_tail():
    case = Case(256, 512, 128, 4, torch.bfloat16, seed=9, bits2=4, bias=True)
    for M in (33, 257):
        x = case.x(M)
        assert rel_err(case.module()(x.cuda()), case.oracle(x)) <= TOL


def test_fused_gate_up_prefill():
    dt = torch.bfloat16
    gate, up = Case(512, 256, 128, 4, dt, seed=4, lut_std=0.05), Case(512, 256, 128, 4, dt, seed=5)
    M = 200
    x = gate.x(M).cuda()
    g, u = gate.module(), up.module()
    u._ensure_packed()
    out = torch.empty(M, 512, dtype=dt, device="cuda")
    d = g._segment_desc(out)
    d.update(packed2=u._packed, lut2=u.lut, bits2=4)
    L.gemm(x, L.make_segments([d]), epilogue=L.EPI_SILU_MUL)
    want = orc.silu_mul_fused(x.cpu().float() @ gate.w1.t(), x.cpu().float() @ up.w1.t(), dt)
    assert rel_err(out, want) <= TOL


def test_two_stream_sub_4_bit_routes_through_the_decode_kernel():
    case = Case(256, 256, 64, 3, torch.float16, seed=12, bits2=2)
    x = case.x(40)
    assert rel_err(case.module()(x.cuda()), case.oracle(x)) <= TOL


def test_prefill_shape_of_the_9b_model_sampled():
    # M = 2048, K = 4096, N = 12288 (gate/up shape): every token, 512 sampled weight rows
    N, K, M, gs = 12288, 4096, 2048, 128
    blob = pkg.synthetic.random_blob_on_device(N, K, 4, 77, "cuda")
    lut = pkg.synthetic.make_lut(N // gs, 4, torch.bfloat16, 77)
    mod = pkg.PalettizedLinear(blob, lut.cuda(), 4, gs, N, K).cuda()
    x = pkg.synthetic.make_x(M, K, torch.bfloat16, 78)
    got = mod(x.cuda())
    rows = torch.cat([torch.arange(t * 128, t * 128 + 128) for t in (0, 37, 70, 95)])
    codes = L.unpack_codes(mod._packed, N, K, 4)[rows.cuda()].cpu().numpy()
    w = torch.empty(len(rows), K)
    for j, r in enumerate(rows.tolist()):
        w[j] = lut[r // gs].float()[torch.from_numpy(codes[j].astype(np.int64))]
    want = (x.float() @ w.t()).to(torch.bfloat16)
    assert rel_err(got[:, rows.cuda()], want) <= TOL
    # the block-rotated variant: same GEMM behind a 128-point Hadamard of the activations
    xr = pkg.fht.fht_block(x.cuda(), 128)
    got_r = mod(xr)
    want_r = (orc.fht_block(x, 128).float() @ w.t()).to(torch.bfloat16)
    assert rel_err(got_r[:, rows.cuda()], want_r) <= TOL


def _raw_gemm(case, mod, x, split, out=None, ldo=None):
    """One call of the C entry on the module's own codes and palettes."""
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, case.N, dtype=case.dtype, device="cuda")
    d = dict(packed=mod._packed, lut=mod.lut, N=case.N, group_size=case.gs,
             n_groups=mod.lut.shape[0], bits=case.bits, out=out, ldo=ldo or out.stride(0))
    if case.bias is not None:
        d["bias"] = case.bias.cuda()
    L.gemm(x, L.make_segments([d]), split=split)
    return out


@pytest.mark.parametrize("N,K,gs,bits,dtype,M,bias", (
    (12288, 1024, 128, 4, torch.bfloat16, 512, True),    # 192 tiles: one full round + 44 cut in 3
    (2560, 512, 128, 4, torch.float16, 300, False),      # 40 tiles, no full round, 108 SMs share them
    (8192, 2048, 64, 4, torch.bfloat16, 513, True),      # token tail: the third tile row holds one token
    (4096, 1024, 128, 3, torch.bfloat16, 1100, False),   # 3-bit codes
    (1280, 256, 128, 2, torch.float16, 256, True),       # short K: parts of two k-blocks
))
def test_split_schedule_equals_the_whole_tile_schedule(N, K, gs, bits, dtype, M, bias):
    assert L.lib().b200lut_gemm_workspace_bytes(M, N, K) > 0
    case = Case(N, K, gs, bits, dtype, seed=N + M, bias=bias)
    mod = case.module()
    mod(case.x(17).cuda())                       # repacks the codes
    x = case.x(M)
    xd = x.cuda()
    whole = _raw_gemm(case, mod, xd, split=False)
    cut = _raw_gemm(case, mod, xd, split=True)
    again = _raw_gemm(case, mod, xd, split=True)     # the counters returned to zero by themselves
    assert torch.equal(cut, again)
    # same products, summed in 2..8 fp32 pieces instead of one: within one rounding of the output
    assert rel_err(cut, whole) <= 2.0 ** -7
    want = case.oracle(x)
    assert rel_err(cut, want) <= TOL and rel_err(whole, want) <= TOL


def test_split_schedule_into_an_unaligned_strided_output():
    N, K, M = 2560, 512, 260
    case = Case(N, K, 128, 4, torch.bfloat16, seed=5, bias=True)
    mod = case.module()
    mod(case.x(17).cuda())
    x = case.x(M)
    buf = torch.full((M, N + 24), 7.0, dtype=torch.bfloat16, device="cuda")
    view = buf[:, 3:3 + N]                       # 6 bytes off the 16-byte grid, row stride N + 24
    _raw_gemm(case, mod, x.cuda(), split=True, out=view)
    assert rel_err(view, case.oracle(x)) <= TOL
    assert (buf[:, :3] == 7.0).all() and (buf[:, 3 + N:] == 7.0).all()


def test_small_or_misaligned_workspace_falls_back_to_whole_tiles():
    N, K, M = 2560, 512, 300
    case = Case(N, K, 128, 4, torch.bfloat16, seed=6)
    mod = case.module()
    mod(case.x(17).cuda())
    x = case.x(M).cuda()
    whole = _raw_gemm(case, mod, x, split=False)
    need = L.lib().b200lut_gemm_workspace_bytes(M, N, K)
    ws = torch.zeros(need + 16, dtype=torch.uint8, device="cuda")
    out = torch.empty_like(whole)
    seg = L.make_segments([dict(packed=mod._packed, lut=mod.lut, N=N, group_size=128,
                                n_groups=mod.lut.shape[0], bits=4, out=out)])
    for ptr, size in ((ws.data_ptr(), need - 1), (ws.data_ptr() + 4, need)):
        out.zero_()
        L.check(L.lib().b200lut_gemm_ws(x.data_ptr(), x.stride(0), M, K, L.dtype_id(x.dtype), seg,
                                        0, 0, ptr, size, L._stream(x)))
        assert torch.equal(out, whole)
    assert not ws.any()                          # the fallback never touched the buffer


@pytest.mark.parametrize("M,N,dtype", ((200, 512, torch.bfloat16), (3, 12288, torch.float16)))
def test_silu_mul_pass(M, N, dtype):
    g = torch.Generator().manual_seed(M + N)
    gate = torch.randn(M, N + 8, generator=g).to(dtype).cuda()[:, :N]      # strided rows
    up = torch.randn(M, N, generator=g).to(dtype).cuda()
    want = (torch.nn.functional.silu(gate.float()) * up.float()).to(dtype)
    got = L.silu_mul(gate, up)
    torch.cuda.synchronize()
    assert rel_err(got, want) <= 2e-3                                       # __expf, one rounding


def test_stack_prefill_step_matches_module_forwards():
    st = __import__("importlib").import_module(pkg.__name__ + ".stack")
    stack = st.LinearStack(n_layers=1)
    M = 96
    x = torch.randn(M, st.HIDDEN, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).cuda()
    plan = stack._plan(M)
    plan["x"].copy_(x)
    y = stack.step(M)
    torch.cuda.synchronize()
    mlp = stack.layers[0].mlp
    want = mlp.down_proj(torch.nn.functional.silu(mlp.gate_proj(x).float()).to(torch.bfloat16) * mlp.up_proj(x))
    assert rel_err(y, want) <= TOL


@pytest.mark.parametrize("M,Ns,K,gs,bits,dtype,bias", (
    (64, (256, 128, 512), 512, 128, 4, torch.bfloat16, True),       # Q/K/V-like, 7 row tiles
    (300, (1024, 1024), 1024, 64, 4, torch.float16, False),         # gate/up-like, token tail
    (40, (128, 128, 128, 256), 256, 128, 3, torch.bfloat16, True),  # four projections, 3-bit
    (2048, (2048, 512), 512, 128, 4, torch.bfloat16, False),        # 160 tiles: one round + cut tiles
    (17, (128, 384), 128, 128, 2, torch.float16, True),
))
def test_merged_prefill_launch_equals_the_separate_launches(M, Ns, K, gs, bits, dtype, bias):
    cases = [Case(N, K, gs, bits, dtype, seed=100 * i + N + M, bias=bias) for i, N in enumerate(Ns)]
    mods = [c.module() for c in cases]
    x = cases[0].x(M)
    xd = x.cuda()
    sep = [m(xd) for m in mods]
    total = sum(Ns)
    out = torch.full((M, total + 8), 5.0, dtype=dtype, device="cuda")
    descs, off = [], 0
    for m in mods:
        descs.append(m._segment_desc(out[:, off:], ldo=total + 8))
        off += m.N
    assert L.gemm_multi_ok(descs, K)
    for split in (True, False):
        out[:, :total] = 0
        L.gemm_multi(xd, L.make_segments(descs), len(descs), split=split)
        off = 0
        for c, m, y in zip(cases, mods, sep):
            got = out[:, off:off + m.N]
            assert rel_err(got, y) <= 2.0 ** -7, (split, off)       # same products, other split of K
            assert rel_err(got, c.oracle(x)) <= TOL
            off += m.N
        assert (out[:, total:] == 5.0).all()


def test_merged_prefill_launch_refuses_mixed_projections():
    a = Case(128, 128, 128, 4, torch.bfloat16, seed=1)
    b = Case(128, 128, 128, 3, torch.bfloat16, seed=2)
    ma, mb = a.module(), b.module()
    x = a.x(32).cuda()
    out = torch.empty(32, 256, dtype=torch.bfloat16, device="cuda")
    descs = [ma._segment_desc(out, ldo=256), mb._segment_desc(out[:, 128:], ldo=256)]
    assert not L.gemm_multi_ok(descs, 128)
    with pytest.raises(RuntimeError, match="share one code width"):
        L.gemm_multi(x, L.make_segments(descs), 2)
    with pytest.raises(RuntimeError, match="nseg"):
        L.gemm_multi(x, L.make_segments(descs * 3), 6)


def test_split_qkv_and_mlp_take_the_merged_prefill_route():
    K, M = 256, 48
    q, k, v = (Case(N, K, 128, 4, torch.bfloat16, seed=N, bias=True) for N in (256, 128, 384))
    qkv = pkg.SplitQKV(q.module(), k.module(), v.module())
    x = q.x(M)
    assert pkg.palettized_modules._prefill_mergeable((qkv.q_proj, qkv.k_proj, qkv.v_proj), x.cuda())
    got = qkv(x.cuda().view(2, 24, K))
    want = torch.cat([c.oracle(x) for c in (q, k, v)], dim=-1)
    assert got.shape == (2, 24, 768) and rel_err(got.reshape(M, -1), want) <= TOL
    g, u, d = (Case(512, K, 128, 4, torch.bfloat16, seed=7), Case(512, K, 128, 4, torch.bfloat16, seed=8),
               Case(K, 512, 128, 4, torch.bfloat16, seed=9))
    mlp = pkg.FusedPalettizedMLP(g.module(), u.module(), d.module(), torch.nn.SiLU())
    y = mlp(x.cuda())
    h = (torch.nn.functional.silu(g.oracle(x).float()) * u.oracle(x).float()).to(torch.bfloat16)
    assert rel_err(y, d.oracle(h)) <= 2 * TOL


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
def test_shapes_and_seeds_of_the_reference_gpu_gate(bits):
    # the reference's standalone GPU gate (src/flute_extended/test_flute.py:133-223): M = 256,
    # K = 512, N = 256, group 32, fp16, A ~ N(0,1), palette ~ N(0,1), codes uniform, seeds 42 and
    # 43 + b; its own kernels are compared bit for bit with each other there — here the result
    # is compared with the oracle (max rel err <= 1e-2, cosine >= 0.999)
    M, K, N, gs = 256, 512, 256, 32
    torch.manual_seed(42 if bits == 4 else 43 + bits)
    A = torch.randn(M, K).half()
    codes = torch.randint(0, 1 << bits, (N, K), dtype=torch.uint8).numpy()
    lut = torch.randn(N // gs, 1 << bits).half()
    mod = pkg.PalettizedLinear(torch.from_numpy(orc.pack_idxn(codes, bits)), lut, bits, gs, N, K).cuda()
    got = mod(A.cuda()).cpu()
    want = orc.linear_forward(A, orc.dequant_indices(codes, lut, gs, bits))
    assert rel_err(got, want) <= TOL
    assert orc.cosine(got.float(), want.float()) >= 0.999
    # the dequantised weights themselves, bit for bit, through the same module
    W = mod(torch.eye(K, dtype=torch.float16, device="cuda")).cpu().t()
    assert torch.equal(W.float(), orc.dequant_indices(codes, lut, gs, bits).float())


@pytest.mark.parametrize("bits,bits2,gs,dtype,N,K,M,bias", (
    (4, 2, 128, torch.bfloat16, 512, 1024, 300, True),     # the deployed mixed-radix pair
    (3, 1, 64, torch.float16, 256, 256, 40, False),
    (2, 4, 128, torch.bfloat16, 384, 512, 129, True),
    (4, 3, 256, torch.bfloat16, 1024, 2048, 2048, False),  # full prefill width
))
def test_two_streams_of_different_widths_on_the_tensor_cores(bits, bits2, gs, dtype, N, K, M, bias):
    case = Case(N, K, gs, bits, dtype, seed=bits * 10 + bits2, bits2=bits2, bias=bias)
    mod = case.module()
    x = case.x(M)
    got = mod(x.cuda())
    want = case.oracle(x)
    assert rel_err(got, want) <= TOL
    # the same module through the decode kernel, 16 rows at a time: one rounding in both routes
    rows = slice(0, 16)
    assert rel_err(got[rows], mod(x[rows].cuda())) <= 2.0 ** -7


def test_two_stream_entry_refuses_a_missing_stream_and_a_small_scratch():
    case = Case(128, 128, 128, 4, torch.bfloat16, seed=3)
    mod = case.module()
    x = case.x(32).cuda()
    out = torch.empty(32, 128, dtype=torch.bfloat16, device="cuda")
    seg = L.make_segments([mod._segment_desc(out)])
    with pytest.raises(RuntimeError, match="second stream"):
        L.gemm_two_stream(x, seg)
    two = Case(128, 128, 128, 4, torch.bfloat16, seed=4, bits2=2).module()
    seg = L.make_segments([two._segment_desc(out)])
    rc = L.lib().b200lut_gemm_two_stream(x.data_ptr(), 128, 32, 128, 0, seg, 0, out.data_ptr(), 64, None)
    assert rc == 4


@pytest.mark.parametrize("N,K,gs,bits,dtype,M,bias", (
    (12288, 1024, 128, 4, torch.bfloat16, 512, True),    # 96 pairs of tiles on 74 pairs of SMs: cut tiles too
    (1024, 2048, 64, 3, torch.float16, 300, False),      # a second token tile 44 rows wide: the halves meet at 32
    (256, 256, 128, 2, torch.bfloat16, 256, True),       # one pair, one tile each
))
def test_cta_pairs_give_the_same_bits_as_single_ctas(N, K, gs, bits, dtype, M, bias):
    """tcgen05 cta_group::2: two CTAs of a cluster run one MMA over 256 weight rows, each holding
    its own 128 rows in tensor memory and half of the activation tile in shared memory. Every
    output element is the same sum in the same order as with one CTA per tile."""
    case = Case(N, K, gs, bits, dtype, seed=N + M, bias=bias)
    mod = case.module()
    mod._ensure_packed()
    x = case.x(M).cuda()
    single = _raw_gemm(case, mod, x, split=False)
    d = dict(packed=mod._packed, lut=mod.lut, N=case.N, group_size=case.gs, n_groups=mod.lut.shape[0],
             bits=case.bits, out=torch.full((M, N), float("nan"), dtype=dtype, device="cuda"))
    if case.bias is not None:
        d["bias"] = case.bias.cuda()
    L.gemm(x, L.make_segments([d]), flags=L.FLAG_CTA_PAIRS, split=False)
    assert torch.equal(d["out"], single)               # whole tiles: the same sums in the same order
    assert rel_err(single, case.oracle(x.cpu())) <= TOL
    d["out"].fill_(float("nan"))
    L.gemm(x, L.make_segments([d]), flags=L.FLAG_CTA_PAIRS)     # cut tiles: other K split points
    assert rel_err(d["out"], single) <= 4e-3
