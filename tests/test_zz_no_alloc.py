"""The allocation-free decode entry (b200lut_gemv_noalloc), called through the C ABI.

It exists for hosts that cannot give the library memory at call time (a fixed device pool,
a no-allocation region, no allocator at all): its split-K scratch is an array inside the
library image. The test checks that it returns what the ordinary entry returns — same
inputs, same split, so the same fp32 fold order — on two calls in a row (the array keeps
the previous call's partials and its tickets must have reset), and that a request beyond
the built-in scratch is refused with a clear message. Collected last on purpose."""
from __future__ import annotations

import pytest
import torch

from helpers import TOL, Case, pkg, rel_err

pytestmark = pytest.mark.gpu
L = pkg._lib


def _call(fn_noalloc, case, mod, x, split):
    out = torch.full((x.shape[0], case.N), float("nan"), dtype=x.dtype, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    did = L.dtype_id(x.dtype)
    if fn_noalloc:
        rc = L.lib().b200lut_gemv_noalloc(x.data_ptr(), mod._packed.data_ptr(), mod.lut.data_ptr(),
                                          out.data_ptr(), x.shape[0], case.N, case.K, case.bits,
                                          case.gs, mod.lut.shape[0], did, split, stream)
    else:
        rc = L.lib().b200lut_gemv(x.data_ptr(), mod._packed.data_ptr(), mod.lut.data_ptr(),
                                  out.data_ptr(), x.shape[0], case.N, case.K, case.bits, case.gs,
                                  mod.lut.shape[0], did, split, None, 0, stream)
    L.check(rc)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("N,K,bits,M,split", ((1024, 2048, 4, 1, 4), (512, 1024, 3, 5, 8),
                                               (2048, 4096, 4, 16, 2)))
def test_noalloc_matches_the_ordinary_entry_twice(N, K, bits, M, split):
    case = Case(N, K, 128, bits, torch.bfloat16, seed=N + M)
    mod = case.module()
    mod._ensure_packed()
    x = case.x(M).cuda()
    want = _call(False, case, mod, x, split)
    first = _call(True, case, mod, x, split)
    second = _call(True, case, mod, x, split)
    for got in (first, second):
        assert not torch.isnan(got.float()).any()
        assert rel_err(got, want) <= TOL
        assert rel_err(got, case.oracle(x.cpu())) <= TOL
    assert torch.equal(first, second)


def test_noalloc_different_shapes_back_to_back_and_reset():
    """Calls of different shapes share the one built-in array: tickets of the first shape must
    be back at zero when the second shape uses the same words, un-split calls (split 1) use no
    scratch at all, a side stream works like the default one, and the reset entry (what a host
    calls after it has recovered from a launch that never finished) leaves the array usable."""
    cases = [(Case(1024, 2048, 128, 4, torch.bfloat16, seed=11), 1, 4),
             (Case(512, 1024, 64, 4, torch.float16, seed=12), 3, 8),
             (Case(2048, 1024, 128, 4, torch.bfloat16, seed=13), 2, 1),
             (Case(1024, 2048, 128, 4, torch.bfloat16, seed=11), 1, 16)]
    prepared = []
    for case, M, split in cases:
        mod = case.module()
        mod._ensure_packed()
        x = case.x(M).cuda()
        ws = None
        if L.gemv_workspace_bytes(case.N, M, split):
            ws = torch.zeros(L.gemv_workspace_bytes(case.N, M, split), dtype=torch.uint8, device="cuda")
        want = torch.empty(M, case.N, dtype=x.dtype, device="cuda")
        L.check(L.lib().b200lut_gemv(x.data_ptr(), mod._packed.data_ptr(), mod.lut.data_ptr(),
                                     want.data_ptr(), M, case.N, case.K, case.bits, case.gs,
                                     mod.lut.shape[0], L.dtype_id(x.dtype), split,
                                     None if ws is None else ws.data_ptr(),
                                     0 if ws is None else ws.numel(), None))
        prepared.append((case, mod, x, split, want))
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    for rounds in range(2):
        for case, mod, x, split, want in prepared:
            got = _call(True, case, mod, x, split)
            assert rel_err(got, case.oracle(x.cpu())) <= TOL
            assert rel_err(got, want) <= TOL
        with torch.cuda.stream(side):
            case, mod, x, split, want = prepared[rounds]
            got = _call(True, case, mod, x, split)
            assert rel_err(got, want) <= TOL
        L.check(L.lib().b200lut_gemv_noalloc_reset(None))
        torch.cuda.synchronize()


def test_noalloc_refuses_what_its_scratch_cannot_hold():
    case = Case(128, 64, 128, 4, torch.bfloat16, seed=1)
    mod = case.module()
    mod._ensure_packed()
    x = case.x(16).cuda()
    out = torch.empty(16, 128, dtype=torch.bfloat16, device="cuda")
    # pretend N = 131072 rows at M = 16, split 16: 16 * 1024 * 16 * 1 KiB = 256 MiB of partials
    rc = L.lib().b200lut_gemv_noalloc(x.data_ptr(), mod._packed.data_ptr(), mod.lut.data_ptr(),
                                      out.data_ptr(), 16, 131072, 1024, 4, 128, 1, L.BF16, 16, None)
    assert rc == 4
    assert b"scratch" in L.lib().b200lut_last_error()
