#!/usr/bin/env python3
"""Benchmark of the B200 LUT-palettized linear path.

Workload (default): the Qwen3.5-9B-shaped linear stack — 248 palettized projections
(6 912 212 992 4-bit weights, group 128, bf16 palettes), one decode step at batch M
(default 1) = one pass of the activation rows through every projection. With N GPUs
the output rows of every projection are sharded column-parallel and the MLP
activation is all-gathered once per layer (strong scaling: total work is fixed).

One JSON line on stdout (rank 0):
  value      tok/s with inputs resident in HBM (CUDA-graph replay of the step)
  e2e        tok/s through the host-facing call: pinned host x -> device, step, result -> host
  roofline   the decode GEMV kernel against the measured HBM copy bandwidth
  cpu_baseline  the CPU oracle (a port of the reference's forward="reference" route)
             timed on this host on a bounded sample, which also checks the GPU outputs
  extras     single-projection GEMV GB/s and (when built) the M=2048 prefill GEMM TFLOP/s

  python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--impl reference]
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG = "rag-cache-engineering-qwen35-9b-flute_b200"
METRIC = "9B linear-stack decode tok/s (LUT-GEMV, M=1 unless --batch)"
FALLBACK_HBM_GBS = 6650.0
DECODE_KERNEL = "gemv_rows_kernel"
TRAFFIC_RATIO = 1.0026
TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one gemv_rows_kernel launch over a "
                  "12288 x 4096 4-bit projection (25.267 MB for 25.202 MB of algorithmic bytes; the "
                  "lm_head-sized launch reads 508.75 MB for 509.13 MB), ratio scaled to the average "
                  "launch of the step")
WORKLOAD = ("qwen3.5-9b linear stack: 32 layers, 248 projections, 6912212992 4-bit weights, "
            "group 128, bf16 palettes")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    return rank, world, local


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def make_gather(world: int, M: int):
    """All-gather of the column-sharded MLP activation [M, world * n] over NCCL."""
    if world == 1:
        return None
    import torch.distributed as dist

    def gather(full, local):
        if M == 1:
            dist.all_gather_into_tensor(full.view(-1), local.reshape(-1))    # in place
        else:
            n = local.shape[1]
            tmp = full.new_empty(world, M, n)
            dist.all_gather_into_tensor(tmp.view(-1), local.contiguous().view(-1))
            full.view(M, world, n).copy_(tmp.permute(1, 0, 2))
    return gather


def time_steps(fn, steps: int, world: int) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the current stream,
    barrier + synchronize on both sides, max over ranks."""
    import torch
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


def cpu_sample(pkg, stack, M: int, gpu_check: bool, threads: int, timed: bool = True, stepped: bool = False):
    """Time the CPU oracle on layers 0 (linear attention) and 3 (full attention) and
    scale to the 24 + 8 layer stack; when gpu_check, compare the GPU outputs of those
    layers with it (max relative error <= 1e-2). On a column-parallel shard (world > 1) the
    oracle computes this rank's rows of every projection; the down projection is checked on the
    activation row the GPU exchange assembled, whose own slice is checked against the oracle.
    timed = False skips the second (cached-indices) timing pass."""
    import numpy as np
    import torch
    from oracle import lut_linear_oracle as orc
    torch.set_num_threads(threads)
    st = importlib.import_module(PKG + ".stack")
    plan = stack._plan(M) if gpu_check else None
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, st.HIDDEN, generator=g).to(stack.dtype)
    if gpu_check and not stepped:     # stepped: the caller already ran the step on check_input()
        plan["x"].copy_(x)
        stack.step(M)
        torch.cuda.synchronize()
    per_kind, worst = {}, 0.0
    for li in [i for i in (0, 3) if i < len(stack.layers)]:
        L = stack.layers[li]
        mods = L.heads() + [L.out(), L.mlp.gate_proj, L.mlp.up_proj, L.mlp.down_proj]
        blobs = [pkg._lib.repack_to_idxn(m._packed, m.N, m.K, m.bitwidth).cpu().numpy() for m in mods]
        luts = [m.lut.cpu() for m in mods]
        t0 = time.perf_counter()
        ys = []
        for m, blob, lut in zip(mods[:-3], blobs, luts):     # as shipped: unpack on every call
            ys.append(orc.linear_forward(x, orc.dequant(blob, lut, m.N, m.K, m.group_size, m.bitwidth)))
        wg, wu, wd = (orc.dequant(b, l, m.N, m.K, m.group_size, m.bitwidth)
                      for m, b, l in zip(mods[-3:], blobs[-3:], luts[-3:]))
        xf = x.float()
        act = orc.silu_mul_fused(xf @ wg.t(), xf @ wu.t(), x.dtype)
        n_loc = act.shape[1]
        down_in = act
        # with a flag-less exchange the consumer refills the rows after use: the multi-GPU gate
        # left its own assembly of them (an NCCL all-gather of the ranks' slices) in the plan
        assembled = plan.get("assembled")
        if stack.world > 1 and gpu_check:      # the full row as the exchange assembled it
            down_in = (assembled[li] if assembled else plan["buffers"][4 * li + 2]).cpu()
        y = orc.linear_forward(down_in, wd)
        per_kind[L.kind] = time.perf_counter() - t0
        if not timed:
            per_kind[L.kind + "_cached"] = per_kind[L.kind]
        # the reference's second mode: logical indices cached once, palette gather per call
        codes = [orc.unpack_idxn(b, m.N, m.K, m.bitwidth) for m, b in zip(mods, blobs)] if timed else None
        t0 = time.perf_counter()
        if timed:
            for m, c, lut in zip(mods[:-3], codes, luts):
                orc.linear_forward(x, orc.dequant_indices(c, lut, m.group_size, m.bitwidth))
            wg2, wu2, wd2 = (orc.dequant_indices(c, l, m.group_size, m.bitwidth)
                             for m, c, l in zip(mods[-3:], codes[-3:], luts[-3:]))
            act2 = orc.silu_mul_fused(xf @ wg2.t(), xf @ wu2.t(), x.dtype)
            orc.linear_forward(act2, wd2)
            per_kind[L.kind + "_cached"] = time.perf_counter() - t0
            del codes, wg2, wu2, wd2
        if gpu_check:
            bufs = plan["buffers"][4 * li:4 * li + 4]
            want_heads = torch.cat(ys[:-1], dim=1)
            act_gpu = (assembled[li] if assembled else bufs[2])[:, stack.rank * n_loc:(stack.rank + 1) * n_loc]
            for got, want in ((bufs[0], want_heads), (bufs[1], ys[-1]), (act_gpu, act), (bufs[3], y)):
                worst = max(worst, orc.max_rel_err(got.cpu().float(), want.float()))
    n_lin = sum(1 for L in stack.layers if L.kind == "linear")
    n_full = len(stack.layers) - n_lin
    per_kind.setdefault("full", per_kind["linear"])
    per_kind.setdefault("full_cached", per_kind["linear_cached"])
    step_s = n_lin * per_kind["linear"] + n_full * per_kind["full"]
    per_kind["step_cached"] = n_lin * per_kind["linear_cached"] + n_full * per_kind["full_cached"]
    return step_s, worst, per_kind


def check_input(stack, M: int):
    """The seeded activation rows the inline correctness gate of the stack runs on."""
    import torch
    st = importlib.import_module(PKG + ".stack")
    return torch.randn(M, st.HIDDEN, generator=torch.Generator().manual_seed(7)).to(stack.dtype)


def exchange_equals_gather(stack, M: int, world: int) -> bool:
    """Multi-GPU gate: after a step, every layer's assembled activation row (filled by the peers'
    stores, or by the NCCL gather) must equal, bit for bit, an NCCL all-gather of the ranks' own
    slices taken now — or, when the exchange consumes the rows (no flags), what the step computed
    from them must equal what it computes from such a gather. True only if it holds on every rank."""
    import torch
    import torch.distributed as dist
    L = importlib.import_module(PKG)._lib
    plan = stack._plan(M)
    ok = True
    if plan.get("sentinel"):
        # Flag-less exchange: the consumer has refilled the rows it consumed, so the check runs on
        # what they produced. Per layer: this rank's slice again (the gate/up launch without the
        # exchange), an NCCL all-gather of the slices, the down launch on the gathered rows without
        # the exchange: its output must equal, bit for bit, what the step left behind. The rows
        # are then marked "not arrived" again for the steps that follow.
        launches = plan["launches"]
        plan["assembled"] = {}
        for li in range(len(stack.layers)):
            _, xin, segs, nseg, epi, _, _, _ = launches[4 * li + 2]
            _, _, dsegs, dn, depi, _, _, _ = launches[4 * li + 3]
            act, y = plan["buffers"][4 * li + 2], plan["buffers"][4 * li + 3]
            y_step = y.clone()
            # (a flag-less exchange always runs the row-range kernel: so do the launches repeated here)
            L.gemv_multi(xin, segs, nseg, epilogue=epi, flags=L.FLAG_ROWS_KERNEL)
            n = act.shape[1] // world
            mine = act[:, stack.rank * n:(stack.rank + 1) * n].contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            full = torch.cat(parts, dim=1)
            L.gemv_multi(full, dsegs, dn, epilogue=depi, flags=L.FLAG_ROWS_KERNEL)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(y, y_step))
            plan["assembled"][li] = full
            act.view(torch.int16).fill_(-1)
        torch.cuda.synchronize()
        dist.barrier()
    else:
        for li in range(len(stack.layers)):
            act = plan["buffers"][4 * li + 2]
            n = act.shape[1] // world
            mine = act[:, stack.rank * n:(stack.rank + 1) * n].contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            ok = ok and bool(torch.equal(torch.cat(parts, dim=1), act))
    act = plan["buffers"][2]
    flag = torch.tensor([1 if ok else 0], device=act.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


GROUPS = ("heads", "out", "gate_up", "down")


def cpu_group_samples(M: int, seed: int):
    """The four projection groups of a linear-attention decoder layer on the CPU oracle (the
    reference's forward="reference" route: numpy unpack of every idxN blob on every call, fp32
    torch matmul): seeded synthetic blobs and palettes drawn on the host. Returns
    {group: (closure that runs the group once, weights of the group)}."""
    import numpy as np
    import torch
    from oracle import lut_linear_oracle as orc
    st = importlib.import_module(PKG + ".stack")
    rng = np.random.default_rng(seed)
    bits, gs = 4, 128

    def make(N, K):
        blob = rng.integers(0, 256, size=N * K * bits // 8, dtype=np.uint8)   # uniform bytes = uniform codes
        g = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
        lut = (0.02 * torch.randn(N // gs, 1 << bits, generator=g)).sort(dim=1).values.to(torch.bfloat16)
        return blob, lut, N, K

    def weight(t):
        return orc.dequant(t[0], t[1], t[2], t[3], gs, bits)
    heads = [make(n, st.HIDDEN) for _, n in st.LINEAR_ATTN]
    out = make(st.HIDDEN, st.HIDDEN)
    gate, up = make(st.INTERMEDIATE, st.HIDDEN), make(st.INTERMEDIATE, st.HIDDEN)
    down = make(st.HIDDEN, st.INTERMEDIATE)
    x = torch.randn(M, st.HIDDEN, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
    act = torch.randn(M, st.INTERMEDIATE, generator=torch.Generator().manual_seed(seed + 1)).to(torch.bfloat16)

    def run_heads():
        for t in heads:
            orc.linear_forward(x, weight(t))

    def run_gate_up():
        xf = x.float()
        return orc.silu_mul_fused(xf @ weight(gate).t(), xf @ weight(up).t(), x.dtype)
    return {"heads": (run_heads, sum(t[2] * t[3] for t in heads)),
            "out": (lambda: orc.linear_forward(x, weight(out)), out[2] * out[3]),
            "gate_up": (run_gate_up, 2 * gate[2] * gate[3]),
            "down": (lambda: orc.linear_forward(act, weight(down)), down[2] * down[3])}


def run_reference(args, rank: int):
    """The reference arm: the CPU oracle (port of the reference's forward="reference" route)
    timed on the host cores with all the threads torch can use. One timed step = ONE projection
    group of a decoder layer (Q/K/V/z heads, out projection, gate + up + SiLU*mul, down
    projection, in turn), so that K steps stay within minutes; the step time of the whole stack
    is the sum over the 128 groups of the 32 layers, each at its group's mean time (the heads of
    the 8 full-attention layers, 10240 rows instead of 12288, by row count)."""
    if rank != 0:
        return
    import torch
    st = importlib.import_module(PKG + ".stack")
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    M = args.batch
    groups = cpu_group_samples(M, 11)
    for i in range(args.warmup):
        groups[GROUPS[i % 4]][0]()
    spent = {g: [] for g in GROUPS}
    t_all = time.perf_counter()
    for i in range(args.steps):
        g = GROUPS[i % 4]
        t0 = time.perf_counter()
        groups[g][0]()
        spent[g].append(time.perf_counter() - t0)
    wall = time.perf_counter() - t_all
    seen = [g for g in GROUPS if spent[g]]
    per_weight = sum(statistics.mean(spent[g]) for g in seen) / sum(groups[g][1] for g in seen)
    mean = {g: statistics.mean(spent[g]) if spent[g] else per_weight * groups[g][1] for g in GROUPS}
    n_lin = sum(1 for i in range(st.N_LAYERS) if st.layer_kind(i) == "linear")
    n_full = st.N_LAYERS - n_lin
    full_heads = sum(n for _, n in st.FULL_ATTN) / sum(n for _, n in st.LINEAR_ATTN)
    step_s = (n_lin + n_full * full_heads) * mean["heads"] + st.N_LAYERS * (mean["out"] + mean["gate_up"] + mean["down"])
    value = M / step_s
    sample = ("each timed step is ONE projection group of a decoder layer on the CPU, in turn: " +
              ", ".join(f"{g} {mean[g]:.2f} s" for g in GROUPS) +
              f"; ms_per_step and value are the 32-layer step = {n_lin} + {n_full} x {full_heads:.3f} heads "
              f"+ {st.N_LAYERS} x (out + gate_up + down)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch": M, "sample": sample, "timed_wall_s": wall},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": f"{args.steps} single-group steps ({wall:.0f} s of CPU work); " + sample +
                                       "; blob unpacked on every call as the reference route does"},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def sampled_gate(pkg, packed, lut, N, K, bits, gs, x, got, rows=None, residual=None):
    """Inline correctness gate of one data point (the reference's benchmark does the same per
    point, src/flute_extended/benchmark_kernel.py:95-107): the outputs of 256 weight rows
    spread over the matrix are recomputed on the CPU with the reference route's arithmetic
    (palette lookup of the exported codes, fp32 matmul, one rounding) and compared. Returns
    {"rel_max": max|got - want| / max|want|, "cos": cosine}; a point with rel_max > 1e-2 or
    cos < 0.999 is not reported."""
    import numpy as np
    import torch
    from oracle import lut_linear_oracle as orc
    if rows is None:
        tiles = sorted({0, (N // 128) // 3, (N // 128) - 1})
        rows = torch.cat([torch.arange(t * 128, min(N, t * 128 + 86)) for t in tiles])[:256]
    codes = pkg._lib.unpack_codes(packed, N, K, bits)[rows.to(packed.device)].cpu().numpy().astype(np.int64)
    lut_c = lut.cpu()
    w = torch.empty(len(rows), K)
    for j, r in enumerate(rows.tolist()):
        w[j] = lut_c[min(r // gs, lut_c.shape[0] - 1)].float()[torch.from_numpy(codes[j])]
    xc = x.detach().cpu()
    want = (xc.float() @ w.t()).to(xc.dtype)
    if residual is not None:      # (resA [N, R], resB [R, K]): the reference route adds it to the rounded sums
        resA, resB = (t.detach().cpu() for t in residual)
        want = want + ((xc @ resB.t()) @ resA[rows].t()).to(want.dtype)
    g = got[:, rows.to(got.device)].detach().cpu()
    return {"rel_max": orc.max_rel_err(g.float(), want.float()), "cos": orc.cosine(g.float(), want.float())}


def gate_ok(g) -> bool:
    return g["rel_max"] <= 1e-2 and g["cos"] >= 0.999


def single_projection_gbs(pkg, M: int, N: int, K: int, sets: int, iters: int, flags: int,
                          bits: int = 4, gs: int = 128, gate: bool = False):
    """Extra: one projection launched back to back over `sets` distinct weight sets
    (their total exceeds L2), CUDA-graph replay; returns (GB/s, us per launch[, gate])."""
    import torch
    L = pkg._lib
    dt = torch.bfloat16
    x = torch.randn(M, K, device="cuda").to(dt)
    out = torch.empty(M, N, dtype=dt, device="cuda")
    keep, segs = [], []
    for i in range(sets):
        packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 900 + i, "cuda"), N, K, bits)
        lut = pkg.synthetic.make_lut(N // gs, bits, dt, 900 + i).cuda()
        keep.append((packed, lut))
        segs.append(L.make_segments([dict(packed=packed, lut=lut, N=N, group_size=gs,
                                          n_groups=N // gs, bits=bits, out=out)]))

    def run():
        for s in segs:
            L.gemv_multi(x, s, 1, flags=flags)
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    for _ in range(3):
        g.replay()
    ms = time_steps(g.replay, iters, 1)
    us = ms * 1e3 / (iters * sets)
    byts = N * K * bits // 8 + (N // gs) * (2 << bits) + M * K * 2 + M * N * 2
    if not gate:
        return byts / us / 1e3, us
    # the graph's last launch used the last weight set: `out` holds its result
    return byts / us / 1e3, us, sampled_gate(pkg, keep[-1][0], keep[-1][1], N, K, bits, gs, x, out)


def prefill_gemm_tflops(pkg, M: int, N: int, K: int, iters: int, rotate: bool, gate: bool = False,
                        rank: int = 0, flags: int = 0):
    """Extra: the M=2048 prefill GEMM (optionally behind the 128-point block Hadamard of the
    activations, or with a rank-`rank` residual: its projection launch and the extra k-block,
    timed together), CUDA events, inputs 16 MB + 24 MB + 48 MB out per call. The FLOP count is
    the code streams' only."""
    import torch
    L = pkg._lib
    bits, gs, dt = 4, 128, torch.bfloat16
    packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 700, "cuda"), N, K, bits)
    lut = pkg.synthetic.make_lut(N // gs, bits, dt, 700).cuda()
    x = torch.randn(M, K, device="cuda").to(dt)
    xr = torch.empty_like(x)
    out = torch.empty(M, N, dtype=dt, device="cuda")
    desc = dict(packed=packed, lut=lut, N=N, group_size=gs, n_groups=N // gs, bits=bits, out=out)
    residual = None
    if rank:
        resA = (0.05 * torch.randn(N, rank, device="cuda")).to(dt)
        resB = (0.05 * torch.randn(rank, K, device="cuda")).to(dt)
        t = torch.empty(M, L.residual_block_cols(rank), dtype=dt, device="cuda")
        desc.update(resA=resA, res_t=t)
        residual = (resA, resB)
    seg = L.make_segments([desc])

    def run():
        if rank:
            L.residual_project_rows(x, resB, out=t)
        if rotate:
            L.fht(x, None, block=128, out=xr)
            L.gemm(xr, seg, flags=flags)
        else:
            L.gemm(x, seg, flags=flags)
    for _ in range(3):
        run()
    ms = time_steps(run, iters, 1)
    status = L.lib().b200lut_device_status()
    if status != 0:
        raise RuntimeError(f"a bounded wait ran out inside the GEMM kernel (device status {status})")
    us = ms * 1e3 / iters
    if not gate:
        return 2.0 * M * N * K / us / 1e6, us
    if rotate:
        from oracle import lut_linear_oracle as orc
        xin = orc.fht_block(x.cpu(), 128).to(dt)
    else:
        xin = x
    return 2.0 * M * N * K / us / 1e6, us, sampled_gate(pkg, packed, lut, N, K, bits, gs, xin[:64], out[:64],
                                                        residual=residual)


def dense_matmul_tflops(M: int, N: int, K: int, iters: int):
    """Extra: the dense bf16 baseline of the same shape (torch.matmul = cuBLAS on a random
    [N, K] bf16 matrix), the comparison the reference's benchmark_kernel.py:171-177 makes."""
    import torch
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (0.02 * torch.randn(N, K, device="cuda")).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")

    def run():
        torch.matmul(x, w.t(), out=out)
    for _ in range(3):
        run()
    us = time_steps(run, iters, 1) * 1e3 / iters
    return 2.0 * M * N * K / us / 1e6, us


def kgrouped_projection_gbs(pkg, M: int, N: int, K: int, sets: int, iters: int, gate: bool = False):
    """Extra: the K-grouped palette variant of one projection (one 16-entry palette per 128
    input columns and output row: N*K/4 bytes of palettes beside N*K/2 of codes), launched
    back to back over `sets` distinct weight sets; returns (GB/s, us per launch)."""
    import torch
    L = pkg._lib
    bits, dt = 4, torch.bfloat16
    x = torch.randn(M, K, device="cuda").to(dt)
    out = torch.empty(M, N, dtype=dt, device="cuda")
    keep = []
    for i in range(sets):
        packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 950 + i, "cuda"), N, K, bits)
        lut_k = (0.02 * torch.randn(K // 128, N, 16, device="cuda",
                                    generator=torch.Generator("cuda").manual_seed(950 + i))).sort(dim=-1).values.to(dt)
        keep.append((packed, lut_k))

    def run():
        for packed, lut_k in keep:
            L.gemv_kgrouped(x, packed, lut_k, N, bits, out=out)
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    for _ in range(3):
        g.replay()
    ms = time_steps(g.replay, iters, 1)
    us = ms * 1e3 / (iters * sets)
    byts = N * K * bits // 8 + (K // 128) * N * 16 * 2 + M * K * 2 + M * N * 2
    if not gate:
        return byts / us / 1e3, us
    # gate: 128 sampled rows of the last weight set, palette per (128-column block, row)
    import numpy as np
    from oracle import lut_linear_oracle as orc
    packed, lut_k = keep[-1]
    rows = torch.arange(0, N, N // 128)[:128]
    codes = L.unpack_codes(packed, N, K, bits)[rows.cuda()].cpu().numpy().astype(np.int64)
    pal = lut_k[:, rows.cuda()].cpu().float()                     # [K/128, rows, 16]
    w = torch.empty(len(rows), K)
    for j in range(len(rows)):
        c = torch.from_numpy(codes[j]).view(K // 128, 128)
        w[j] = pal[:, j].gather(1, c).reshape(K)
    want = (x.cpu().float() @ w.t()).to(dt)
    got = out[:, rows.cuda()].cpu()
    return byts / us / 1e3, us, {"rel_max": orc.max_rel_err(got.float(), want.float()),
                                 "cos": orc.cosine(got.float(), want.float())}


def kgrouped_gemm_tflops(pkg, M: int, N: int, K: int, iters: int):
    """Extra: the K-grouped palette variant at prefill width on the tensor cores
    (b200lut_gemm_kgrouped); returns (TFLOP/s, us, gate on 128 sampled weight rows x 64 tokens)."""
    import numpy as np
    import torch
    from oracle import lut_linear_oracle as orc
    L = pkg._lib
    bits, dt = 4, torch.bfloat16
    packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 970, "cuda"), N, K, bits)
    lut_k = (0.02 * torch.randn(K // 128, N, 16, device="cuda",
                                generator=torch.Generator("cuda").manual_seed(970))).sort(dim=-1).values.to(dt)
    x = torch.randn(M, K, device="cuda").to(dt)
    out = torch.empty(M, N, dtype=dt, device="cuda")

    def run():
        L.gemm_kgrouped(x, packed, lut_k, N, bits, out=out)
    for _ in range(3):
        run()
    us = time_steps(run, iters, 1) * 1e3 / iters
    if L.lib().b200lut_device_status() != 0:
        raise RuntimeError("a bounded wait ran out inside the K-grouped GEMM")
    rows = torch.arange(0, N, N // 128)[:128]
    codes = L.unpack_codes(packed, N, K, bits)[rows.cuda()].cpu().numpy().astype(np.int64)
    pal = lut_k[:, rows.cuda()].cpu().float()
    w = torch.empty(len(rows), K)
    for j in range(len(rows)):
        w[j] = pal[:, j].gather(1, torch.from_numpy(codes[j]).view(K // 128, 128)).reshape(K)
    want = (x[:64].cpu().float() @ w.t()).to(dt)
    got = out[:64][:, rows.cuda()].cpu()
    return 2.0 * M * N * K / us / 1e6, us, {"rel_max": orc.max_rel_err(got.float(), want.float()),
                                            "cos": orc.cosine(got.float(), want.float())}


def embedding_gather_gbs(pkg, N: int, K: int, n_ids: int, iters: int, gate: bool = False):
    """Extra: the embedding gather over an lm_head-sized 4-bit table (0.51 GB of codes, far
    beyond L2), `n_ids` random rows per launch; returns (GB/s of algorithmic bytes, us).
    Algorithmic bytes per row: K/2 of codes + 2K of output."""
    import torch
    L = pkg._lib
    bits, gs, dt = 4, 128, torch.bfloat16
    packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 811, "cuda"), N, K, bits)
    lut = pkg.synthetic.make_lut(N // gs, bits, dt, 811).cuda()
    table = dict(packed=packed, lut=lut, bits=bits, N=N, group_size=gs, n_groups=N // gs)
    # 16 launches per graph replay, each with its own ids and output rows: 64 MB of code sectors
    # and 268 MB of output per replay, beyond L2 (an eager call is bound by the host: 18-20 us)
    gen = torch.Generator("cuda").manual_seed(5)
    sets = [(torch.randint(0, N, (n_ids,), device="cuda", generator=gen),
             torch.empty(n_ids, K, dtype=dt, device="cuda")) for _ in range(16)]
    ids = sets[0][0]

    def run():
        for i, o in sets:
            L.embed_gather(i, table, K, dt, out=o)
    for _ in range(3):
        run()
    us = graph_time(run, iters) / len(sets)
    if L.lib().b200lut_device_status() != 0:
        raise RuntimeError("the embedding gather met an id outside its table")
    if not gate:
        return n_ids * (K * bits // 8 + 2 * K) / us / 1e3, us
    # gate: the gathered rows equal the palette lookup of the exported codes, bit for bit
    # (the weight rows come from the dequant export of the 128-row tiles that hold them)
    rows = L.embed_gather(ids[:8].contiguous(), table, K, dt)
    tile_bytes = 128 * K * bits // 8
    exact = True
    for j, i in enumerate(ids[:8].tolist()):
        t = i // 128
        w = L.dequant(packed[t * tile_bytes:(t + 1) * tile_bytes], lut[t * 128 // gs:(t + 1) * 128 // gs].contiguous(),
                      128, K, bits, gs)
        exact = exact and bool(torch.equal(rows[j], w[i % 128]))
    return n_ids * (K * bits // 8 + 2 * K) / us / 1e3, us, {"bit_exact": exact}


def graph_time(run, iters: int):
    """us per call of `run` under CUDA-graph replay (one eager call first)."""
    import torch
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    for _ in range(3):
        g.replay()
    return time_steps(g.replay, iters, 1) * 1e3 / iters


def projection_point(pkg, M: int, N: int, K: int, bits: int, gs: int, iters: int, flags: int):
    """One point of the hybrid-palettization grid: the module forward of one projection (decode
    GEMV at M <= 16, tensor-core GEMM above) over enough distinct weight sets to exceed L2,
    CUDA-graph replay. Returns (us per forward, algorithmic bytes, gate)."""
    import torch
    dt = torch.bfloat16
    sets = max(2, -(-160_000_000 // (N * K * bits // 8)))
    x = torch.randn(M, K, device="cuda").to(dt)
    mods = []
    for i in range(sets):
        packed = pkg._lib.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 300 + i, "cuda"), N, K, bits)
        lut = pkg.synthetic.make_lut(N // gs, bits, dt, 300 + i).cuda()
        mods.append(pkg.PalettizedLinear.from_packed(packed, lut, bits, gs, N, K))
    outs = [None]

    def run():
        for m in mods:
            outs[0] = m(x)
    pkg.set_programmatic_launch(bool(flags & pkg._lib.FLAG_PDL))
    us = graph_time(run, iters) / sets
    byts = N * K * bits // 8 + (N // gs) * (2 << bits) + M * K * 2 + M * N * 2
    last = mods[-1]
    return us, byts, sampled_gate(pkg, last._packed, last.lut, N, K, bits, gs, x, outs[0])


def mlp_block_point(pkg, M: int, form: str, iters: int, flags: int):
    """The decode MLP block (gate, up 4096 -> 12288; SiLU*mul; down 12288 -> 4096) in one of three
    forms over 4 weight sets (300 MB of codes): "plain" = gate, up, one SiLU*mul pass, down as
    four launches with the library's launch shapes; "split" = the same with the K split of the
    tile kernel set by hand (2 for gate / up, 8 for down: the reference's split-K form);
    "fused" = gate + up + SiLU*mul in one launch, then down. Returns (us per block, gate)."""
    import torch
    L = pkg._lib
    dt, H, I, bits, gs = torch.bfloat16, 4096, 12288, 4, 128
    x = torch.randn(M, H, device="cuda").to(dt)
    sets = []
    for i in range(4):
        mk = lambda N, K, sd: (L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, sd, "cuda"), N, K, bits),
                               pkg.synthetic.make_lut(N // gs, bits, dt, sd).cuda())
        sets.append((mk(I, H, 500 + 3 * i), mk(I, H, 501 + 3 * i), mk(H, I, 502 + 3 * i)))
    g_out = torch.empty(M, I, dtype=dt, device="cuda")
    u_out = torch.empty(M, I, dtype=dt, device="cuda")
    y = torch.empty(M, H, dtype=dt, device="cuda")

    def seg(w, N, out):
        return dict(packed=w[0], lut=w[1], N=N, group_size=gs, n_groups=N // gs, bits=bits, out=out)
    prepared = []
    for g, u, d in sets:
        prepared.append((L.make_segments([seg(g, I, g_out)]), L.make_segments([seg(u, I, u_out)]),
                         L.make_segments([seg(g, I, g_out), seg(u, I, None)]), L.make_segments([seg(d, H, y)])))

    def run():
        for sg, su, sgu, sd in prepared:
            if form == "fused":
                L.gemv_multi(x, sgu, 2, epilogue=L.EPI_SILU_MUL, flags=flags)
            else:
                kw = dict(split=2, flags=flags | L.FLAG_TILE_KERNEL) if form == "split" else dict(flags=flags)
                L.gemv_multi(x, sg, 1, **kw)
                L.gemv_multi(x, su, 1, **kw)
                L.silu_mul(g_out, u_out)
            kw = dict(split=8, flags=flags | L.FLAG_TILE_KERNEL) if form == "split" else dict(flags=flags)
            L.gemv_multi(g_out, sd, 1, **kw)
    us = graph_time(run, iters) / len(sets)
    # gate: the activation row on sampled gate / up rows, then down on the GPU's own activation row
    from oracle import lut_linear_oracle as orc
    g, u, d = sets[-1]
    rows = torch.arange(0, I, I // 128)[:128]
    import numpy as np

    def wrows(w, N, K, r):
        codes = L.unpack_codes(w[0], N, K, bits)[r.cuda()].cpu().numpy().astype(np.int64)
        lut = w[1].cpu().float()
        return torch.stack([lut[rr // gs][torch.from_numpy(codes[j])] for j, rr in enumerate(r.tolist())])
    xf = x.cpu().float()
    act_want = orc.silu_mul_fused(xf @ wrows(g, I, H, rows).t(), xf @ wrows(u, I, H, rows).t(), dt)
    act_got = g_out[:, rows.cuda()].cpu()
    gate_act = {"rel_max": orc.max_rel_err(act_got.float(), act_want.float()),
                "cos": orc.cosine(act_got.float(), act_want.float())}
    gate_y = sampled_gate(pkg, d[0], d[1], H, I, bits, gs, g_out, y)
    return us, {"rel_max": max(gate_act["rel_max"], gate_y["rel_max"]), "cos": min(gate_act["cos"], gate_y["cos"])}


def stack_point(pkg, stack, M: int, flags: int, iters: int):
    """The stack at batch M under CUDA-graph replay: (ms per step, gate on layer 0's Q rows)."""
    import torch
    plan = stack._plan(M)
    x = torch.randn(M, plan["x"].shape[1], generator=torch.Generator().manual_seed(40 + M)).to(stack.dtype)
    plan["x"].copy_(x)
    ms = graph_time(lambda: stack.step(M, flags=flags), iters) / 1e3
    q = stack.layers[0].heads()[0]
    xin = x
    if stack.rotate:
        from oracle import lut_linear_oracle as orc
        signs = plan["rotated"][0].cpu()
        xin = orc.fht_forward(x, signs)
    got = plan["buffers"][0][:, :q.N]
    return ms, sampled_gate(pkg, q._packed, q.lut, q.N, q.K, q.bitwidth, q.group_size, xin, got)


def run_extras(pkg, st, stack, peaks, flags):
    """Driver-run numbers beside the headline, each behind its own inline correctness gate (a
    point that fails its gate is reported as failed, without a number)."""
    import torch
    extras = {}
    hbm = peaks["hbm_gbs"]

    def put(name, entry, gate):
        if gate is not None and not (gate.get("bit_exact") if "bit_exact" in gate else gate_ok(gate)):
            extras[name] = {"failed_gate": gate}
        else:
            if gate is not None:
                entry["gate"] = gate
            extras[name] = entry
    try:
        tf, us, g = prefill_gemm_tflops(pkg, 2048, 12288, 4096, 20, False, gate=True)
        put("prefill_gemm_m2048_k4096_n12288", {
            "TFLOP/s": tf, "us": us, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
            "peak": peaks["bf16_tflops"], "peak_kind": "burst, " + peaks["source"]}, g)
        dtf, dus = dense_matmul_tflops(2048, 12288, 4096, 20)
        extras["dense_bf16_matmul_m2048_k4096_n12288"] = {"TFLOP/s": dtf, "us": dus, "lut_gemm_over_dense": tf / dtf}
        tf, us, g = prefill_gemm_tflops(pkg, 2048, 12288, 4096, 20, True, gate=True)
        put("prefill_gemm_with_block128_fht", {"TFLOP/s": tf, "us": us, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}, g)
        tf, us, g = prefill_gemm_tflops(pkg, 2048, 12288, 4096, 20, False, gate=True, rank=32)
        put("prefill_gemm_with_rank32_residual", {"TFLOP/s": tf, "us": us, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
                                                   "launches": "residual_rows_kernel + gemm_tc_persistent_kernel"}, g)
        for name, N, K, sets, it in (("gemv_4096x4096_m1", 4096, 4096, 40, 20), ("gemv_12288x4096_m1", 12288, 4096, 16, 20),
                                     ("gemv_4096x12288_m1", 4096, 12288, 16, 20),
                                     # the model's lm_head (0.51 GB of codes): the kernel's steady-state rate
                                     ("gemv_248320x4096_m1_lm_head", 248320, 4096, 1, 10)):
            gbs, us, g = single_projection_gbs(pkg, 1, N, K, sets, it, flags, gate=True)
            put(name, {"GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / hbm}, g)
        gbs, us, g = kgrouped_projection_gbs(pkg, 1, 4096, 4096, 16, 20, gate=True)
        put("gemv_kgrouped_4096x4096_m1", {"GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / hbm,
                                            "bytes_per_launch": 12599296}, g)
        gbs, us, g = kgrouped_projection_gbs(pkg, 8, 4096, 4096, 16, 20, gate=True)
        put("gemv_kgrouped_4096x4096_m8", {"GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / hbm}, g)
        tf, us, g = kgrouped_gemm_tflops(pkg, 2048, 12288, 4096, 20)
        put("prefill_gemm_kgrouped_m2048_k4096_n12288", {"TFLOP/s": tf, "us": us,
                                                          "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}, g)
        gbs, us, g = embedding_gather_gbs(pkg, 248320, 4096, 2048, 20, gate=True)
        put("embedding_gather_248320x4096_2048_ids", {"GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / hbm}, g)

        # the decode MLP block: 75.5 MB of algorithmic bytes per block
        mlp_bytes = 3 * (12288 * 4096 // 2) + 2 * (12288 // 128) * 32 + (4096 // 128) * 32
        for M in (1, 8):
            for form in ("plain", "split", "fused"):
                us, g = mlp_block_point(pkg, M, form, 10, flags)
                byts = mlp_bytes + M * (2 * 4096 + 2 * 12288 * 2 + 2 * 4096)
                put(f"mlp_block_m{M}_{form}", {"us_per_block": us, "GB/s": byts / us / 1e3,
                                               "frac_of_hbm": byts / us / 1e3 / hbm}, g)

        # the hybrid-palettization grid: code width x group size x batch on the two projection shapes
        grid = {}
        for N in (4096, 12288):
            for bits in (3, 4):
                for gs in (64, 128):
                    for M in (1, 16, 128):
                        us, byts, g = projection_point(pkg, M, N, 4096, bits, gs, 10, flags)
                        key = f"{N}x4096_b{bits}_gs{gs}_m{M}"
                        if gate_ok(g):
                            grid[key] = {"us": round(us, 2), "frac_of_hbm": round(byts / us / 1e3 / hbm, 3),
                                         "TFLOP/s": round(2.0 * M * N * 4096 / us / 1e6, 1), "rel_max": g["rel_max"]}
                        else:
                            grid[key] = {"failed_gate": g}
        extras["hybrid_grid"] = grid

        # the stack at the other decode widths, and behind a Hadamard rotation of every group's input
        for M in (4, 8, 16, 64):
            ms, g = stack_point(pkg, stack, M, flags, 10)
            byts = stack.algorithmic_bytes(M)
            put(f"stack_m{M}", {"ms_per_step": ms, "tok/s": M * 1e3 / ms, "frac_of_hbm": byts / (ms * 1e-3) / 1e9 / hbm,
                                "launches_per_step": stack.launches_per_step(M)}, g)
        rot = st.LinearStack(device=stack.device, n_layers=len(stack.layers), rotate=True)
        ms, g = stack_point(pkg, rot, 1, flags, 10)
        put("stack_m1_rotated", {"ms_per_step": ms, "tok/s": 1e3 / ms, "launches_per_step": rot.launches_per_step(1),
                                 "note": "one FHT launch (segments + signs) in front of each of the 128 projection groups"}, g)
        del rot
        rot = st.LinearStack(device=stack.device, n_layers=len(stack.layers), rotate="fused")
        ms, g = stack_point(pkg, rot, 1, flags, 10)
        put("stack_m1_rotated_fused", {"ms_per_step": ms, "tok/s": 1e3 / ms, "launches_per_step": rot.launches_per_step(1),
                                       "note": "the rotation runs inside each decode launch (b200lut_gemv_input)"}, g)
        del rot
        torch.cuda.empty_cache()

        # the whole stack at prefill width: every projection as a tensor-core GEMM, eager launches
        Mp = 2048
        ms_p, g = None, None
        stack._plan(Mp)["x"].copy_(torch.randn(Mp, 4096, generator=torch.Generator().manual_seed(77)).to(stack.dtype))
        stack.step(Mp)
        torch.cuda.synchronize()
        ms_p = time_steps(lambda: stack.step(Mp), 5, 1) / 5
        tf_p = stack.flops(Mp) / (ms_p * 1e-3) / 1e12
        q = stack.layers[0].heads()[0]
        plan = stack._plan(Mp)
        g = sampled_gate(pkg, q._packed, q.lut, q.N, q.K, q.bitwidth, q.group_size, plan["x"][:64], plan["buffers"][0][:64, :q.N])
        put("prefill_stack_m2048", {"tok/s": Mp * 1e3 / ms_p, "ms_per_step": ms_p, "TFLOP/s": tf_p,
                                    "frac_of_bf16_peak_sustained": tf_p / peaks["bf16_tflops_sustained"],
                                    "peak_sustained": peaks["bf16_tflops_sustained"]}, g)
        if pkg._lib.lib().b200lut_device_status() != 0:
            raise RuntimeError("a bounded wait ran out inside an extra")
    except Exception as e:       # an extra must not lose the main line
        extras["error"] = repr(e)
    return extras


def run_case(args) -> int:
    """A few eager launches of one kernel on a profiling-sized case. gemv: 12288 x 4096
    4-bit projection at M = 1 over 8 distinct weight sets (192 MB of codes, larger than L2);
    gemv_head: one 248320 x 4096 projection (the kernel's steady state);
    gemm: M = 2048, K = 4096, N = 12288; embed: 2048 rows of an lm_head-sized table."""
    import torch
    torch.cuda.set_device(0)
    pkg = importlib.import_module(PKG)
    peaks = measured_peaks()
    if args.case == "gemv":
        gbs, us = single_projection_gbs(pkg, args.batch, 12288, 4096, 8, max(args.steps, 1), 0)
        print(json.dumps({"case": "gemv 12288x4096 M=%d, 8 weight sets" % args.batch, "GB/s": gbs,
                          "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    elif args.case == "gemv_head":
        gbs, us = single_projection_gbs(pkg, args.batch, 248320, 4096, 1, max(args.steps, 1), 0)
        print(json.dumps({"case": "gemv 248320x4096 (lm_head size, 0.51 GB of codes) M=%d" % args.batch,
                          "GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    elif args.case == "kgrouped":
        gbs, us = kgrouped_projection_gbs(pkg, args.batch, 4096, 4096, 16, max(args.steps, 1))
        print(json.dumps({"case": "K-grouped gemv 4096x4096 M=%d, 16 weight sets" % args.batch, "GB/s": gbs,
                          "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    elif args.case == "embed":
        gbs, us = embedding_gather_gbs(pkg, 248320, 4096, 2048, max(args.steps, 1))
        print(json.dumps({"case": "embedding gather, 2048 rows of a 248320 x 4096 4-bit table",
                          "GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    else:
        pairs = args.case == "gemm_pairs"
        rank = 32 if args.case == "gemm_res" else 0
        tf, us = prefill_gemm_tflops(pkg, 2048, 12288, 4096, max(args.steps, 1), False, rank=rank,
                                     flags=pkg._lib.FLAG_CTA_PAIRS if pairs else 0)
        print(json.dumps({"case": "gemm M=2048 K=4096 N=12288" + (", CTA pairs (cta_group::2)" if pairs else "")
                          + (", rank-32 residual (projection launch + residual k-blocks)" if rank else ""),
                          "TFLOP/s": tf, "us": us, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch (1/0)")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the stack (32 = the model)")
    ap.add_argument("--gather", choices=("push", "nccl"), default="push",
                    help="N > 1: how the sharded MLP activation is recombined (push: peer stores "
                         "from the GEMV epilogue; nccl: an all-gather call between the launches)")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a graph replay")
    ap.add_argument("--case", default="stack", choices=("stack", "gemv", "gemv_head", "gemm", "gemm_pairs", "gemm_res", "embed", "kgrouped"),
                    help="stack: the benchmark; gemv / gemv_head / gemm / gemm_pairs / gemm_res / embed / "
                         "kgrouped: a few launches of one kernel on a profiling-sized case")
    ap.add_argument("--executor", default="graph", choices=("plan", "graph"),
                    help="plan: persistent cooperative launch(es) per step; graph: one kernel per "
                         "projection group under CUDA-graph replay")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")))
        return 0

    import torch
    if args.case != "stack":
        return run_case(args)
    rank, world, local = dist_setup(args.gpus)
    pkg = importlib.import_module(PKG)
    st = importlib.import_module(PKG + ".stack")
    M = args.batch
    flags = pkg._lib.FLAG_PDL if args.pdl else 0
    peaks = measured_peaks()

    push = world > 1 and args.gather == "push" and M <= 16 and args.executor != "plan"
    stack = st.LinearStack(device=f"cuda:{local}", rank=rank, world=world, n_layers=args.layers,
                           gather="push" if push else "nccl")
    gather = make_gather(world, M)
    plan = stack._plan(M)
    x_host = torch.randn(M, st.HIDDEN, generator=torch.Generator().manual_seed(1)).to(stack.dtype).pin_memory()
    y_host = torch.empty(plan["y"].shape, dtype=stack.dtype).pin_memory()
    plan["x"].copy_(x_host)

    # eager run, then capture the step in a CUDA graph
    use_plan = args.executor == "plan" and M <= 16

    def run_step():
        if use_plan:
            stack.step_persistent(M, gather=gather)
        else:
            stack.step(M, flags=flags, gather=gather)
    if world > 1:
        # ranks reach this point at different times (allocation, page locking); the exchange
        # waits inside the kernels are bounded, so line the ranks up before the first step
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
    run_step()
    torch.cuda.synchronize()
    # Inline correctness gate of the timed configuration, on every rank count: one eager step on
    # seeded rows; rank 0 compares its rows of layers 0 and 3 with the CPU oracle below, and with
    # several ranks the assembled activation rows must equal an NCCL all-gather bit for bit.
    plan["x"].copy_(check_input(stack, M))
    run_step()
    torch.cuda.synchronize()
    multi_gpu_check = None
    if world > 1:
        multi_gpu_check = {"assembled_rows_equal_nccl_all_gather": exchange_equals_gather(stack, M, world)}
    gate_worst = None
    if rank == 0 and not args.no_cpu and world > 1:
        _, gate_worst, _ = cpu_sample(pkg, stack, M, True, os.cpu_count() or 1, timed=False, stepped=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    plan["x"].copy_(x_host)
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            run_step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            # thread-local capture: the NCCL watchdog thread keeps making CUDA calls of its own
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                run_step()
        torch.cuda.synchronize()

    def step_resident():
        if graph is not None:
            graph.replay()
        else:
            run_step()

    def step_e2e():
        plan["x"].copy_(x_host, non_blocking=True)
        step_resident()
        y_host.copy_(plan["y"], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(args.warmup):
        step_resident()
    with ClockSampler(local) as clk:
        # run under load for ~1.5 s first so that the 200 ms sampler sees the timed state,
        # then time exactly K steps
        probe_ms = time_steps(step_resident, args.steps, world)
        for _ in range(min(int(1500 / max(probe_ms, 1e-3)), 200)):
            for _ in range(args.steps):
                step_resident()
        ms = time_steps(step_resident, args.steps, world)
    clocks = clk.summary()
    for _ in range(args.warmup):
        step_e2e()
    ms_e2e = time_steps(step_e2e, args.steps, world)

    status = pkg._lib.lib().b200lut_device_status()
    if status != 0:
        raise RuntimeError(f"rank {rank}: a bounded device wait ran out (status {status:#x}); "
                           "the timings are void")
    ms_step = ms / args.steps
    tok_s = M * 1e3 / ms_step
    launches = stack.launches_per_step(M)
    kernel_launches = sum(1 for k, _ in stack.decode_plans(M) if k == "plan") if use_plan else launches
    bytes_rank = stack.algorithmic_bytes(M)
    achieved = bytes_rank / (ms_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "batch": M,
                   "parallelism": f"column-parallel x{world}, all-gather of the MLP activation per layer" + (
                       "" if world == 1 else
                       " folded into the GEMV launches (peer stores over NVLink + flag wait)" if push
                       else " (NCCL)") + (
                       "" if world == 1 else
                       "; the other sharded outputs (heads, out, down) have no full-K consumer in the "
                       "stack and stay sharded, so the result read back is this rank's 1/N of y"),
                   "l2": "inputs (3.46 GB of codes per step) exceed the 126 MB L2",
                   "launch": ("persistent cooperative launch per step (jobs chained by completion counters; "
                              + "/".join(sorted({p.form for k, p in stack.decode_plans(M) if k == "plan"}))
                              + " form), CUDA graph replay" if use_plan else
                              "one kernel per projection group, CUDA graph replay"
                              + (", programmatic dependent launch" if args.pdl else ""))},
        "e2e": {"value": M * 1e3 / (ms_e2e / args.steps), "unit": "tok/s",
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
        "gpu_launches": kernel_launches * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "gemv_plan_kernel" if use_plan else DECODE_KERNEL, "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "peak_source": peaks["source"],
                     # DRAM bytes per launch: the ncu capture of this kernel read TRAFFIC_RATIO times
                     # the algorithmic bytes of its launch and wrote none; traffic grows with the
                     # codes, so the ratio is applied to the average launch of the step
                     "traffic": None if use_plan else TRAFFIC_RATIO * bytes_rank / kernel_launches,
                     "traffic_source": TRAFFIC_SOURCE,
                     "bytes_per_launch": bytes_rank / kernel_launches,
                     "us_per_launch": ms_step * 1e3 / kernel_launches,
                     "projection_groups_per_step": launches},
    }
    if M > 64:
        # beyond the crossover the step is bound by the tensor cores: report it against the
        # sustained bf16 peak (the kernel is timed inside a long step)
        tf = stack.flops(M) / (ms_step * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "kernel": "gemm_tc_persistent_kernel", "achieved": tf,
                            "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                            "frac": tf / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"],
                            "traffic": None, "flops_per_step": stack.flops(M),
                            "us_per_launch": ms_step * 1e3 / kernel_launches,
                            "projection_groups_per_step": launches}
    if rank == 0 and world == 1 and not args.no_extras:
        line["extras"] = run_extras(pkg, st, stack, peaks, flags)
    if multi_gpu_check is not None:
        line["multi_gpu_check"] = multi_gpu_check
        if gate_worst is not None:
            line["multi_gpu_check"]["gpu_max_rel_err_vs_cpu"] = gate_worst
            line["multi_gpu_check"]["checked"] = "rank 0's rows of layers 0 and 3 against the CPU oracle"
        if not multi_gpu_check["assembled_rows_equal_nccl_all_gather"] or (gate_worst or 0.0) > 1e-2:
            line["invalid"] = "multi-GPU outputs differ from the NCCL gather or from the CPU oracle"
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        step_s, worst, per_kind = cpu_sample(pkg, stack, M, True, threads)
        line["cpu_baseline"] = {
            "value": M / step_s, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"layers 0 (linear-attention, {per_kind['linear']:.1f} s) and 3 "
                      f"(full-attention, {per_kind['full']:.1f} s), scaled x24 + x8; blob unpacked "
                      "on every call as the reference route does",
            "value_with_cached_indices": M / per_kind["step_cached"],
            "gpu_max_rel_err_vs_cpu": worst}
        if worst > 1e-2:
            line["invalid"] = f"GPU outputs differ from the CPU oracle: max rel err {worst}"
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # A captured graph that holds NCCL work keeps the communicator busy; tearing the
        # process group down under it can block. Everything is reported: drop the graph,
        # meet the other ranks once more and leave without the teardown.
        import torch.distributed as dist
        del graph
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
