"""Column-parallel exchange folded into the decode GEMV (push all-gather).

Single GPU: two "ranks" live on one device, each with its own arena; their launches are
issued in the order gate_up(0), gate_up(1), down(0), down(1), ..., so every flag a launch
waits for has been raised by a launch that completed before it started (nothing waits on
a later launch). The recombined activation and the outputs must equal, bit for bit, a
manual gather of the same shards, and match the unsharded stack within the output
tolerance. Two GPUs (skipped on fewer): the same through real peer mappings, one process
per GPU, against the NCCL all-gather.
"""
from __future__ import annotations

import os
import sys

import pytest
import torch

from helpers import TOL, pkg, rel_err

pytestmark = pytest.mark.gpu
stack_mod = __import__("importlib").import_module(pkg.__name__ + ".stack")
exchange = __import__("importlib").import_module(pkg.__name__ + ".exchange")


def _emulated_step(stacks, M, x):
    plans = [s._plan(M) for s in stacks]
    for p in plans:
        p["x"].copy_(x)
    for entries in zip(*[p["launches"] for p in plans]):
        for s, e in zip(stacks, entries):
            s.run_launch(e, M)
    torch.cuda.synchronize()
    return plans


@pytest.mark.parametrize("M,world", ((1, 2), (5, 2), (1, 8), (3, 4)))
def test_emulated_ranks_push_equals_manual_gather(M, world):
    layers = 2
    arenas = exchange.PeerArena.emulated(1 << 20, world, "cuda")
    pushed = [stack_mod.LinearStack(n_layers=layers, rank=r, world=world, gather="push",
                                    arenas=arenas[r]) for r in range(world)]
    manual = [stack_mod.LinearStack(n_layers=layers, rank=r, world=world, gather="nccl")
              for r in range(world)]
    x = torch.randn(M, stack_mod.HIDDEN, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()

    for rep in range(3):      # the flags and tickets must be reusable step after step
        plans = _emulated_step(pushed, M, x)
        assert pkg._lib.lib().b200lut_device_status() == 0

        # manual gather: run both shards launch by launch, copying slices at the gather entries
        mplans = [s._plan(M) for s in manual]
        for p in mplans:
            p["x"].copy_(x)
        for entries in zip(*[p["launches"] for p in mplans]):
            if entries[0][0] == "gather":
                for r, e in enumerate(entries):
                    n = e[2].shape[1]
                    for q in range(world):
                        if q != r:
                            entries[q][1][:, r * n:(r + 1) * n].copy_(e[2])
                continue
            for s, e in zip(manual, entries):
                # a flag-less exchange always runs the row-range kernel; the launches it is
                # compared with, bit for bit, must run the same one
                s.run_launch(e, M, pkg._lib.FLAG_ROWS_KERNEL if plans[0]["sentinel"] else 0)
        torch.cuda.synchronize()
        for r in range(world):
            for i, (got, want) in enumerate(zip(plans[r]["buffers"], mplans[r]["buffers"])):
                if plans[r]["sentinel"] and i % 4 == 2:
                    # a flag-less exchange consumes the rows: the consumer has marked them "not
                    # arrived" again; what it computed from them is the next buffer
                    assert bool((got.view(torch.int16) == -1).all())
                    continue
                assert torch.equal(got, want), f"rank {r}, repetition {rep}, buffer {i}"

    full = stack_mod.LinearStack(n_layers=layers)
    fp = full._plan(M)
    fp["x"].copy_(x)
    y = full.step(M)
    torch.cuda.synchronize()
    n = y.shape[1] // world
    for r in range(world):
        assert rel_err(plans[r]["y"].float().cpu(), y[:, r * n:(r + 1) * n].float().cpu()) <= TOL


def test_push_needs_two_layers():
    with pytest.raises(ValueError):
        stack_mod.LinearStack(n_layers=1, rank=0, world=2, gather="push")


def _two_gpu_worker(rank, world, port, ok, M):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    layers = 3
    a = stack_mod.LinearStack(device=f"cuda:{rank}", n_layers=layers, rank=rank, world=world, gather="push")
    b = stack_mod.LinearStack(device=f"cuda:{rank}", n_layers=layers, rank=rank, world=world, gather="nccl")
    x = torch.randn(M, stack_mod.HIDDEN, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()

    def gather(full, local):
        parts = [torch.empty_like(local.contiguous()) for _ in range(world)]
        dist.all_gather(parts, local.contiguous())
        full.copy_(torch.cat(parts, dim=1))
    bad = 0     # bit 0: a buffer differs, 1: consumed rows not refilled, 2: y differs, 3: device status
    for _ in range(4):
        a._plan(M)["x"].copy_(x)
        b._plan(M)["x"].copy_(x)
        ya = a.step(M, flags=pkg._lib.FLAG_PDL)
        yb = b.step(M, flags=pkg._lib.FLAG_ROWS_KERNEL if a._plan(M)["sentinel"] else 0, gather=gather)
        torch.cuda.synchronize()
        consumed = a._plan(M)["sentinel"]      # a flag-less exchange refills the rows it has consumed
        for i, (p, q) in enumerate(zip(a._plan(M)["buffers"], b._plan(M)["buffers"])):
            if consumed and i % 4 == 2:
                bad |= 0 if bool((p.view(torch.int16) == -1).all()) else 2
            else:
                bad |= 0 if torch.equal(p, q) else 1
        bad |= 0 if torch.equal(ya, yb) else 4
        torch.cuda.synchronize()
        dist.barrier()       # the peer's next push must not land while this rank still looks at its rows
    bad |= 0 if pkg._lib.lib().b200lut_device_status() == 0 else 8
    dist.barrier()
    ok[rank] = 1 if bad == 0 else -bad
    a._plan(M)["arena"].close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one box")
@pytest.mark.parametrize("M", (1, 6))      # without flags (the rows are their own signal), with flags
def test_two_gpu_push_equals_nccl_gather(M):
    import torch.multiprocessing as mp
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_two_gpu_worker, args=(world, 29531 + M, ok, M), nprocs=world, join=True)
    assert list(ok) == [1] * world


def test_a_wait_that_runs_out_returns_reports_the_rank_and_the_channel_recovers():
    """Nothing pushes, so the consumer's flag wait runs out at its (here 1 ms) bound: the launch
    still returns, the device status names the rank whose flag was missing, later waits do not
    block, and after the host has read the status and re-zeroed the exchange words a complete
    push / wait round gives the plain result."""
    from helpers import Case
    L = pkg._lib
    dt, M, world = torch.bfloat16, 1, 2
    arenas = exchange.PeerArena.emulated(1 << 16, world, "cuda")
    prods = [Case(128, 256, 128, 4, dt, seed=90 + r) for r in range(world)]
    cons = Case(128, 256, 128, 4, dt, seed=95)
    pmods = [c.module() for c in prods]
    cmod = cons.module()
    for m in pmods + [cmod]:
        m._ensure_packed()
    x = prods[0].x(M).cuda()
    blocks = L.gemv_launch_blocks(M, 256, L.make_segments([pmods[0]._segment_desc(None)]), 1)
    chans = [exchange.Channel(arenas[r], M, 256, dt, blocks) for r in range(world)]
    out = torch.zeros(M, cons.N, dtype=dt, device="cuda")
    csegs = L.make_segments([cmod._segment_desc(out)])

    # the same without flags: the rows start as 0xFFFF and nothing replaces them
    sarenas = exchange.PeerArena.emulated(1 << 16, world, "cuda")
    schans = [exchange.Channel(sarenas[r], M, 256, dt, blocks, sentinel=True) for r in range(world)]
    schans[0].wait.wait_ms = 1
    L.gemv_exchange(schans[0].act, csegs, 1, schans[0].wait)
    torch.cuda.synchronize()
    status = L.lib().b200lut_device_status()
    assert status in (0x7000, 0x7001), hex(status)
    assert bool((schans[0].act.view(torch.int16) == -1).all())   # refilled (it never changed) for the next round
    for rep in range(2):
        for r in range(world):
            dst = schans[r].act[:, r * 128:(r + 1) * 128]
            L.gemv_exchange(x, L.make_segments([pmods[r]._segment_desc(dst, ldo=256)]), 1, schans[r].push)
        L.gemv_exchange(schans[0].act, csegs, 1, schans[0].wait)
        L.gemv_exchange(schans[1].act, csegs, 1, schans[1].wait)
        torch.cuda.synchronize()
        assert L.lib().b200lut_device_status() == 0
        assert torch.equal(out, cmod(torch.cat([m(x) for m in pmods], dim=1)))
        assert bool((schans[0].act.view(torch.int16) == -1).all())   # the consumer's last block refilled the rows

    chans[0].wait.wait_ms = 1
    L.gemv_exchange(chans[0].act, csegs, 1, chans[0].wait)      # no producer has run
    L.gemv_exchange(chans[0].act, csegs, 1, chans[0].wait)      # the status is sticky: returns at once
    torch.cuda.synchronize()
    status = L.lib().b200lut_device_status()
    assert status in (0x7000, 0x7001), hex(status)              # 0x7000 + a rank whose flag was missing
    assert L.lib().b200lut_device_status() == 0                 # reading it cleared it

    for a in arenas:                                            # recovery: counters and flags back to zero
        a.buf.zero_()
    for rep in range(2):
        for r in range(world):
            dst = chans[r].act[:, r * 128:(r + 1) * 128]
            L.gemv_exchange(x, L.make_segments([pmods[r]._segment_desc(dst, ldo=256)]), 1, chans[r].push)
        L.gemv_exchange(chans[0].act, csegs, 1, chans[0].wait)
        torch.cuda.synchronize()
        assert L.lib().b200lut_device_status() == 0
        act = torch.cat([m(x) for m in pmods], dim=1)
        assert torch.equal(chans[0].act, act) and torch.equal(chans[1].act, act)
        assert torch.equal(out, cmod(act))
