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


def cpu_sample(pkg, stack, M: int, gpu_check: bool, threads: int):
    """Time the CPU oracle on layers 0 (linear attention) and 3 (full attention) and
    scale to the 24 + 8 layer stack; when gpu_check, compare the GPU outputs of those
    layers with it (max relative error <= 1e-2)."""
    import numpy as np
    import torch
    from oracle import lut_linear_oracle as orc
    torch.set_num_threads(threads)
    st = importlib.import_module(PKG + ".stack")
    plan = stack._plan(M) if gpu_check else None
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, st.HIDDEN, generator=g).to(stack.dtype)
    if gpu_check:
        plan["x"].copy_(x)
        stack.step(M)
        torch.cuda.synchronize()
    per_kind, worst = {}, 0.0
    for li in (0, 3):
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
        y = orc.linear_forward(act, wd)
        per_kind[L.kind] = time.perf_counter() - t0
        # the reference's second mode: logical indices cached once, palette gather per call
        codes = [orc.unpack_idxn(b, m.N, m.K, m.bitwidth) for m, b in zip(mods, blobs)]
        t0 = time.perf_counter()
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
            for got, want in ((bufs[0], want_heads), (bufs[1], ys[-1]), (bufs[2], act), (bufs[3], y)):
                worst = max(worst, orc.max_rel_err(got.cpu().float(), want.float()))
    n_lin = sum(1 for L in stack.layers if L.kind == "linear")
    n_full = len(stack.layers) - n_lin
    step_s = n_lin * per_kind["linear"] + n_full * per_kind["full"]
    per_kind["step_cached"] = n_lin * per_kind["linear_cached"] + n_full * per_kind["full_cached"]
    return step_s, worst, per_kind


def run_reference(args, rank: int):
    """The reference arm: the CPU oracle (port of the reference's forward="reference"
    route: numpy unpack of the idxN blob on every call, fp32 torch matmul) timed on
    the host cores. One step = one 4096 x 4096 projection; tok/s is scaled to the
    stack by the weight ratio."""
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import lut_linear_oracle as orc
    pkg = importlib.import_module(PKG)
    st = importlib.import_module(PKG + ".stack")
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    M, N, K, bits, gs = args.batch, 4096, 4096, 4, 128
    codes, blob = pkg.synthetic.make_blob(N, K, bits, pkg.synthetic.BASE_SEED)
    lut = pkg.synthetic.make_lut(N // gs, bits, torch.bfloat16, pkg.synthetic.BASE_SEED)
    x = pkg.synthetic.make_x(M, K, torch.bfloat16, pkg.synthetic.BASE_SEED)
    blob = blob.numpy()

    def step():
        return orc.linear_forward(x, orc.dequant(blob, lut, N, K, gs, bits))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    scale = st.census()["weights"] / (N * K)
    value = M / (dt * scale)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * scale * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "qwen3.5-9b linear stack: 32 layers, 248 projections, 6912212992 4-bit weights, group 128, bf16 palettes",
                       "batch": M},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": f"one 4096x4096 projection per step ({dt * 1e3:.0f} ms), "
                                       f"scaled x{scale:.0f} by weight count"},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def single_projection_gbs(pkg, M: int, N: int, K: int, sets: int, iters: int, flags: int):
    """Extra: one projection launched back to back over `sets` distinct weight sets
    (their total exceeds L2), CUDA-graph replay; returns (GB/s, us per launch)."""
    import torch
    L = pkg._lib
    bits, gs, dt = 4, 128, torch.bfloat16
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
    byts = N * K * bits // 8 + (N // gs) * 32 + M * K * 2 + M * N * 2
    return byts / us / 1e3, us


def prefill_gemm_tflops(pkg, M: int, N: int, K: int, iters: int, rotate: bool):
    """Extra: the M=2048 prefill GEMM (optionally behind the 128-point block Hadamard of the
    activations, timed together), CUDA events, inputs 16 MB + 24 MB + 48 MB out per call."""
    import torch
    L = pkg._lib
    bits, gs, dt = 4, 128, torch.bfloat16
    packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 700, "cuda"), N, K, bits)
    lut = pkg.synthetic.make_lut(N // gs, bits, dt, 700).cuda()
    x = torch.randn(M, K, device="cuda").to(dt)
    xr = torch.empty_like(x)
    out = torch.empty(M, N, dtype=dt, device="cuda")
    seg = L.make_segments([dict(packed=packed, lut=lut, N=N, group_size=gs, n_groups=N // gs,
                                bits=bits, out=out)])

    def run():
        if rotate:
            L.fht(x, None, block=128, out=xr)
            L.gemm(xr, seg)
        else:
            L.gemm(x, seg)
    for _ in range(3):
        run()
    ms = time_steps(run, iters, 1)
    status = L.lib().b200lut_device_status()
    if status != 0:
        raise RuntimeError(f"a bounded wait ran out inside the GEMM kernel (device status {status})")
    us = ms * 1e3 / iters
    return 2.0 * M * N * K / us / 1e6, us


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


def kgrouped_projection_gbs(pkg, M: int, N: int, K: int, sets: int, iters: int):
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
    return byts / us / 1e3, us


def embedding_gather_gbs(pkg, N: int, K: int, n_ids: int, iters: int):
    """Extra: the embedding gather over an lm_head-sized 4-bit table (0.51 GB of codes, far
    beyond L2), `n_ids` random rows per launch; returns (GB/s of algorithmic bytes, us).
    Algorithmic bytes per row: K/2 of codes + 2K of output."""
    import torch
    L = pkg._lib
    bits, gs, dt = 4, 128, torch.bfloat16
    packed = L.repack_from_idxn(pkg.synthetic.random_blob_on_device(N, K, bits, 811, "cuda"), N, K, bits)
    lut = pkg.synthetic.make_lut(N // gs, bits, dt, 811).cuda()
    table = dict(packed=packed, lut=lut, bits=bits, N=N, group_size=gs, n_groups=N // gs)
    ids = torch.randint(0, N, (n_ids,), device="cuda", generator=torch.Generator("cuda").manual_seed(5))

    def run():
        L.embed_gather(ids, table, K, dt)
    for _ in range(3):
        run()
    ms = time_steps(run, iters, 1)
    if L.lib().b200lut_device_status() != 0:
        raise RuntimeError("the embedding gather met an id outside its table")
    us = ms * 1e3 / iters
    return n_ids * (K * bits // 8 + 2 * K) / us / 1e3, us


def run_case(args) -> int:
    """A few eager launches of one kernel on a profiling-sized case. gemv: 12288 x 4096
    4-bit projection at M = 1 over 8 distinct weight sets (192 MB of codes, larger than L2);
    gemm: M = 2048, K = 4096, N = 12288; embed: 2048 rows of an lm_head-sized table."""
    import torch
    torch.cuda.set_device(0)
    pkg = importlib.import_module(PKG)
    peaks = measured_peaks()
    if args.case == "gemv":
        gbs, us = single_projection_gbs(pkg, args.batch, 12288, 4096, 8, max(args.steps, 1), 0)
        print(json.dumps({"case": "gemv 12288x4096 M=%d, 8 weight sets" % args.batch, "GB/s": gbs,
                          "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    elif args.case == "kgrouped":
        gbs, us = kgrouped_projection_gbs(pkg, args.batch, 4096, 4096, 16, max(args.steps, 1))
        print(json.dumps({"case": "K-grouped gemv 4096x4096 M=%d, 16 weight sets" % args.batch, "GB/s": gbs,
                          "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    elif args.case == "embed":
        gbs, us = embedding_gather_gbs(pkg, 248320, 4096, 2048, max(args.steps, 1))
        print(json.dumps({"case": "embedding gather, 2048 rows of a 248320 x 4096 4-bit table",
                          "GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}))
    else:
        tf, us = prefill_gemm_tflops(pkg, 2048, 12288, 4096, max(args.steps, 1), False)
        print(json.dumps({"case": "gemm M=2048 K=4096 N=12288", "TFLOP/s": tf, "us": us,
                          "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}))
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
    ap.add_argument("--case", default="stack", choices=("stack", "gemv", "gemm", "embed", "kgrouped"),
                    help="stack: the benchmark; gemv / gemm: a few launches of one kernel on a "
                         "small case (the workloads the ncu captures in profiles/ use)")
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

    def trace(msg):
        if os.environ.get("B200LUT_BENCH_TRACE"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)
    trace("building the stack")
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
    trace("first eager step")
    run_step()
    torch.cuda.synchronize()
    trace("eager step done")
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            run_step()
            torch.cuda.synchronize()
            trace("capturing")
            graph = torch.cuda.CUDAGraph()
            # thread-local capture: the NCCL watchdog thread keeps making CUDA calls of its own
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                run_step()
        torch.cuda.synchronize()
        trace("captured")

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
    trace("warm-up done")
    with ClockSampler(local) as clk:
        # run under load for ~1.5 s first so that the 200 ms sampler sees the timed state,
        # then time exactly K steps
        probe_ms = time_steps(step_resident, args.steps, world)
        for _ in range(min(int(1500 / max(probe_ms, 1e-3)), 200)):
            for _ in range(args.steps):
                step_resident()
        ms = time_steps(step_resident, args.steps, world)
    clocks = clk.summary()
    trace("timed")
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
        "config": {"workload": "qwen3.5-9b linear stack: 32 layers, 248 projections, "
                               "6912212992 4-bit weights, group 128, bf16 palettes",
                   "batch": M,
                   "parallelism": f"column-parallel x{world}, all-gather per layer" + (
                       "" if world == 1 else
                       " folded into the GEMV launches (peer stores over NVLink + flag wait)" if push
                       else " (NCCL)"),
                   "l2": "inputs (3.46 GB of codes per step) exceed the 126 MB L2",
                   "launch": ("persistent cooperative launch per step (jobs chained by completion counters), "
                              "CUDA graph replay" if use_plan else
                              "one kernel per projection group, CUDA graph replay"
                              + (", programmatic dependent launch" if args.pdl else ""))},
        "e2e": {"value": M * 1e3 / (ms_e2e / args.steps), "unit": "tok/s",
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
        "gpu_launches": kernel_launches * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "gemv_plan_kernel" if use_plan else "gemv_kernel", "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "peak_source": peaks["source"],
                     # DRAM bytes per launch: the ncu capture of this kernel on the 12288 x 4096
                     # projection read 25.25 MB for 25.20 MB of algorithmic bytes and wrote none
                     # (profiles/gemv_kernel_12288x4096_m1.md); traffic grows with the codes, so
                     # the ratio is applied to the average launch of the step
                     "traffic": None if use_plan else 1.002 * bytes_rank / kernel_launches,
                     "traffic_source": "ncu dram__bytes ratio 1.002 of the 12288x4096 capture, scaled",
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
        extras = {}
        try:
            tf, us = prefill_gemm_tflops(pkg, 2048, 12288, 4096, 20, False)
            extras["prefill_gemm_m2048_k4096_n12288"] = {
                "TFLOP/s": tf, "us": us, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
                "peak": peaks["bf16_tflops"], "peak_kind": "burst, " + peaks["source"]}
            dtf, dus = dense_matmul_tflops(2048, 12288, 4096, 20)
            extras["dense_bf16_matmul_m2048_k4096_n12288"] = {"TFLOP/s": dtf, "us": dus,
                                                              "lut_gemm_over_dense": tf / dtf}
            tf, us = prefill_gemm_tflops(pkg, 2048, 12288, 4096, 20, True)
            extras["prefill_gemm_with_block128_fht"] = {
                "TFLOP/s": tf, "us": us, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}
            gbs, us = single_projection_gbs(pkg, 1, 4096, 4096, 40, 20, flags)
            extras["gemv_4096x4096_m1"] = {"GB/s": gbs, "us_per_launch": us,
                                           "frac_of_hbm": gbs / peaks["hbm_gbs"]}
            gbs, us = single_projection_gbs(pkg, 1, 12288, 4096, 16, 20, flags)
            extras["gemv_12288x4096_m1"] = {"GB/s": gbs, "us_per_launch": us,
                                            "frac_of_hbm": gbs / peaks["hbm_gbs"]}
            # the model's lm_head (248 320 x 4096, 1940 tiles, 0.51 GB of codes): the steady-state
            # streaming rate of the kernel, with the per-launch cost amortised over 13 waves
            gbs, us = single_projection_gbs(pkg, 1, 248320, 4096, 1, 10, flags)
            extras["gemv_248320x4096_m1_lm_head"] = {"GB/s": gbs, "us_per_launch": us,
                                                     "frac_of_hbm": gbs / peaks["hbm_gbs"]}
            gbs, us = kgrouped_projection_gbs(pkg, 1, 4096, 4096, 16, 20)
            extras["gemv_kgrouped_4096x4096_m1"] = {"GB/s": gbs, "us_per_launch": us,
                                                    "frac_of_hbm": gbs / peaks["hbm_gbs"],
                                                    "bytes_per_launch": 12599296}
            gbs, us = embedding_gather_gbs(pkg, 248320, 4096, 2048, 20)
            extras["embedding_gather_248320x4096_2048_ids"] = {
                "GB/s": gbs, "us_per_launch": us, "frac_of_hbm": gbs / peaks["hbm_gbs"]}
            # the whole stack at prefill width: every projection as a tensor-core GEMM
            # (gate, then up multiplying silu of the gate's output), eager launches
            Mp = 2048
            stack.step(Mp)
            torch.cuda.synchronize()
            ms_p = time_steps(lambda: stack.step(Mp), 5, 1) / 5
            tf_p = stack.flops(Mp) / (ms_p * 1e-3) / 1e12
            extras["prefill_stack_m2048"] = {
                "tok/s": Mp * 1e3 / ms_p, "ms_per_step": ms_p, "TFLOP/s": tf_p,
                "frac_of_bf16_peak_sustained": tf_p / peaks["bf16_tflops_sustained"],
                "peak_sustained": peaks["bf16_tflops_sustained"]}
            if pkg._lib.lib().b200lut_device_status() != 0:
                raise RuntimeError("a bounded wait ran out inside the prefill stack")
        except Exception as e:       # an extra must not lose the main line
            extras["error"] = repr(e)
        line["extras"] = extras
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
