"""Synthetic Qwen3.5-9B-shaped linear stack: every palettized projection of the 32
decoder layers, random-init, run as one decode (or prefill) step.

The reference builds its model from a checkpoint (load_palettized_model,
src/scripts/palettized_modules.py:3264-3398); no checkpoint travels with this
package, so this module offers the constructor the reference lacks: the module
census of src/docs/MODEL_GEOMETRY.md (24 linear-attention layers with in_proj_qkv
as Q 2048 + K 2048 + V 4096 rows, in_proj_z 4096, out_proj 4096; 8 full-attention
layers with q 8192, k 1024, v 1024, o 4096; every layer an MLP 4096 -> 12288 ->
4096), 248 modules, 6 912 212 992 weights, 4-bit codes, group 128.

Attention, recurrence, norms and residual adds are excluded (they are not part of
the palettized linear path): every projection group of a step reads the step's
activation rows x [M, 4096]; the MLP chain gate/up -> SiLU*mul -> down is real.

Column-parallel sharding: rank r of G owns output rows [r*N/G, (r+1)*N/G) of every
projection (contiguous bytes in the tile-major code buffer). Sharded outputs that
feed a full-K consumer are recombined with an all-gather (the MLP's SiLU*mul
output before down_proj): either an NCCL call between the two launches, or — decode,
`gather="push"` — folded into them (exchange.py: the gate/up launch stores its slice
into every rank's buffer over NVLink, the down launch waits for the flags).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.nn as nn

from . import _lib, exchange, synthetic
from .palettized_modules import FusedPalettizedMLP, PalettizedLinear, SplitQKV

HIDDEN = 4096
INTERMEDIATE = 12288
N_LAYERS = 32
FULL_ATTENTION_EVERY = 4          # layers 3, 7, ... are full attention (8 of 32)
LINEAR_ATTN = (("q", 2048), ("k", 2048), ("v", 4096), ("z", 4096))
FULL_ATTN = (("q", 8192), ("k", 1024), ("v", 1024))


def layer_kind(i: int) -> str:
    return "full" if (i + 1) % FULL_ATTENTION_EVERY == 0 else "linear"


def census() -> dict:
    """Module and weight counts of the stack (checked against the model geometry)."""
    modules = weights = 0
    for i in range(N_LAYERS):
        heads = LINEAR_ATTN if layer_kind(i) == "linear" else FULL_ATTN
        rows = [n for _, n in heads] + [HIDDEN]                # + out_proj / o_proj
        modules += len(rows) + 3
        weights += sum(rows) * HIDDEN + 3 * INTERMEDIATE * HIDDEN
    return {"modules": modules, "weights": weights}


def shard_rows(N: int, group_size: int, rank: int, world: int):
    """Output rows [lo, hi) of rank `rank`: whole 128-row tiles and whole palette groups."""
    n_loc = N // world
    if N % (world * 128) or (n_loc % group_size and group_size % n_loc):
        raise ValueError(f"N={N} does not shard over {world} ranks in whole tiles and groups")
    return rank * n_loc, (rank + 1) * n_loc


def shard_blob(blob, N: int, K: int, bits: int, rank: int, world: int):
    """Column-parallel shard of an idxN blob: the blob is tile-major over 128-row tiles,
    so the rows of a rank are one contiguous byte range."""
    lo, hi = shard_rows(N, 128, rank, world)
    row_bytes = K * bits // 8
    return blob[lo * row_bytes:hi * row_bytes]


def shard_lut(lut, N: int, group_size: int, rank: int, world: int):
    """Palette rows that serve the rank's output rows."""
    lo, hi = shard_rows(N, group_size, rank, world)
    return lut[lo // group_size:max(hi // group_size, lo // group_size + 1)]


class _Layer(nn.Module):
    def __init__(self, kind: str, mods: dict):
        super().__init__()
        self.kind = kind
        if kind == "linear":
            self.in_proj_qkv = SplitQKV(mods["q"], mods["k"], mods["v"])
            self.in_proj_z = mods["z"]
            self.out_proj = mods["o"]
        else:
            self.qkv = SplitQKV(mods["q"], mods["k"], mods["v"])
            self.o_proj = mods["o"]
        self.mlp = FusedPalettizedMLP(mods["gate"], mods["up"], mods["down"], nn.SiLU())

    def heads(self) -> List[PalettizedLinear]:
        if self.kind == "linear":
            q = self.in_proj_qkv
            return [q.q_proj, q.k_proj, q.v_proj, self.in_proj_z]
        return [self.qkv.q_proj, self.qkv.k_proj, self.qkv.v_proj]

    def out(self) -> PalettizedLinear:
        return self.out_proj if self.kind == "linear" else self.o_proj


class LinearStack(nn.Module):
    """The 32-layer projection stack, optionally one column-parallel shard of it."""

    def __init__(self, device="cuda", dtype=torch.bfloat16, bits: int = 4, group_size: int = 128,
                 n_layers: int = N_LAYERS, seed: int = synthetic.BASE_SEED + 5,
                 rank: int = 0, world: int = 1, gather: str = "nccl", arenas=None,
                 rotate: bool = False):
        super().__init__()
        if gather not in ("nccl", "push"):
            raise ValueError(f"gather must be 'nccl' or 'push', got {gather!r}")
        if gather == "push" and world > 1 and n_layers < 2:
            # with one buffer a peer's next push could overtake this rank's reader
            raise ValueError("gather='push' needs at least two layers")
        self.gather_mode = gather if world > 1 else "nccl"
        # rotate: every projection group reads the Hadamard rotation of its input row (the
        # boundary fold of the reference's rotated artifacts, src/flute_extended/fht.py:105-134),
        # signs drawn per group. True / "launch": one FHT launch in front of each group;
        # "fused": the rotation runs inside the decode launch (M <= 8)
        if rotate not in (False, True, "launch", "fused"):
            raise ValueError(f"rotate must be False, True, 'launch' or 'fused', got {rotate!r}")
        self.rotate = "launch" if rotate is True else rotate
        self.merge_prefill = True    # M > 16: projections that share x run as one launch
        self._arenas = arenas        # test form: pre-built emulated arenas (this rank's one)
        self.device, self.dtype = torch.device(device), dtype
        self.bits, self.group_size = bits, group_size
        self.rank, self.world = rank, world
        self.layers = nn.ModuleList()
        mod_id = 0
        for i in range(n_layers):
            kind = layer_kind(i)
            heads = LINEAR_ATTN if kind == "linear" else FULL_ATTN
            shapes = [(name, n, HIDDEN) for name, n in heads] + [
                ("o", HIDDEN, HIDDEN), ("gate", INTERMEDIATE, HIDDEN),
                ("up", INTERMEDIATE, HIDDEN), ("down", HIDDEN, INTERMEDIATE)]
            mods = {}
            for name, n, k in shapes:
                mods[name] = self._make_module(n, k, seed * 1000 + mod_id)
                mod_id += 1
            self.layers.append(_Layer(kind, mods))
        self._plans = {}

    def _make_module(self, N: int, K: int, seed: int) -> PalettizedLinear:
        """Full-size codes and palette are drawn from the seed (distinct bytes per
        module); a shard keeps rows [rank*N/world, (rank+1)*N/world)."""
        n_loc = N // self.world
        blob = synthetic.random_blob_on_device(N, K, self.bits, seed, self.device)
        blob = shard_blob(blob, N, K, self.bits, self.rank, self.world)
        packed = _lib.repack_from_idxn(blob, n_loc, K, self.bits)
        lut = synthetic.make_lut(N // self.group_size, self.bits, self.dtype, seed)
        lut = shard_lut(lut, N, self.group_size, self.rank, self.world).contiguous().to(self.device)
        return PalettizedLinear.from_packed(packed, lut, self.bits, self.group_size, n_loc, K)

    # ------------------------------------------------------------------ census
    def modules_list(self) -> List[PalettizedLinear]:
        out = []
        for L in self.layers:
            out += L.heads() + [L.out(), L.mlp.gate_proj, L.mlp.up_proj, L.mlp.down_proj]
        return out

    def weight_count(self) -> int:
        return sum(m.N * m.K for m in self.modules_list())

    def algorithmic_bytes(self, M: int) -> int:
        """Bytes one step must move on this rank: codes + palettes + activations in
        and out of every launch (2 bytes per activation element)."""
        total = 0
        for m in self.modules_list():
            total += m.N * m.K * m.bitwidth // 8 + m.lut.numel() * 2 + M * m.K * 2 + M * m.N * 2
        return total

    def flops(self, M: int) -> int:
        return 2 * M * self.weight_count()

    # -------------------------------------------------------------------- step
    def _plan(self, M: int):
        """Persistent buffers and prebuilt segment tables for batch M (stable
        pointers, so a step can be captured in a CUDA graph)."""
        plan = self._plans.get(M)
        if plan is not None:
            return plan
        dev, dt = self.device, self.dtype
        x = torch.zeros(M, HIDDEN, dtype=dt, device=dev)
        launches = []
        outs = []
        push = self.gather_mode == "push" and M <= 16
        sentinel = push and M <= 4 and os.environ.get("B200LUT_EXCHANGE", "").strip() != "flags"
        arena = None
        if push:
            width = self.layers[0].mlp.gate_proj.N * self.world
            need = len(self.layers) * (((M * width * 2 + 255) // 256 + 2) * 256 + self.world * 4096 * 4)
            arena = self._arenas if self._arenas is not None else exchange.PeerArena(
                need, self.rank, self.world, dev)
        fused_rot = self.rotate == "fused" and M <= 8

        def rotated(src, tag):
            """The group's input and its input transform: with launch rotation an ("fht", src,
            dst, signs) entry goes in front and the group reads dst; fused, the group reads src
            through an input transform."""
            if not self.rotate:
                return src, None
            K = src.shape[1]
            g = torch.Generator().manual_seed(len(launches) * 7919 + K)
            signs = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).float().to(dev)
            outs_rot.append(signs)
            if fused_rot:
                return src, _lib.make_input(rot_signs=signs)
            dst = torch.empty_like(src)
            launches.append(("fht", src, dst, signs, None, None, None, None))
            outs_rot.append(dst)
            return dst, None
        outs_rot = []
        for L in self.layers:
            heads = L.heads()
            total = sum(m.N for m in heads)
            hbuf = torch.empty(M, total, dtype=dt, device=dev)
            descs, off = [], 0
            for m in heads:
                descs.append(m._segment_desc(hbuf[:, off:], ldo=total))
                off += m.N
            xr, inp = rotated(x, "heads")
            launches.append(("heads", xr, _lib.make_segments(descs), len(descs), _lib.EPI_NONE, descs, None, inp))
            o = L.out()
            obuf = torch.empty(M, o.N, dtype=dt, device=dev)
            od = [o._segment_desc(obuf)]
            xr, inp = rotated(x, "out")
            launches.append(("out", xr, _lib.make_segments(od), 1, _lib.EPI_NONE, od, None, inp))
            g, u, d = L.mlp.gate_proj, L.mlp.up_proj, L.mlp.down_proj
            chan = None
            if push:
                probe = _lib.make_segments([g._segment_desc(None), u._segment_desc(None)])
                # up to four rows both launches run the row-range kernel, which can take the rows
                # themselves as the arrival signal (no flags, no system-wide fence on the producer)
                chan = exchange.Channel(arena, M, g.N * self.world, dt,
                                        _lib.gemv_launch_blocks(M, g.K, probe, 2, _lib.EPI_SILU_MUL),
                                        sentinel=sentinel)
            act = chan.act if push else torch.empty(M, g.N * self.world, dtype=dt, device=dev)
            act_loc = act[:, self.rank * g.N:(self.rank + 1) * g.N]   # full width after gather
            gd = [g._segment_desc(act_loc, ldo=act.shape[1]), u._segment_desc(None)]
            xr, inp = rotated(x, "gate_up")
            launches.append(("gate_up", xr, _lib.make_segments(gd), 2, _lib.EPI_SILU_MUL, gd,
                             chan.push if push else None, inp))
            if self.world > 1 and not push:
                launches.append(("gather", act, act_loc, None, None, None, None, None))
            ybuf = torch.empty(M, d.N, dtype=dt, device=dev)
            dd = [d._segment_desc(ybuf)]
            if self.rotate and push:
                raise ValueError("a rotated stack uses the NCCL gather (the rotation reads the gathered row)")
            xr, inp = rotated(act, "down")
            launches.append(("down", xr, _lib.make_segments(dd), 1, _lib.EPI_NONE, dd,
                             chan.wait if push else None, inp))
            outs += [hbuf, obuf, act, ybuf]
        if push and sentinel:
            arena.ready(dev)
        plan = {"x": x, "launches": launches, "buffers": outs, "y": outs[-1], "arena": arena,
                "sentinel": bool(push and sentinel),
                "rotated": outs_rot}
        self._plans[M] = plan
        return plan

    def run_launch(self, entry, M: int, flags: int = 0, gather=None) -> None:
        """Issue one entry of the plan's launch list on the current stream."""
        name, xin, segs, nseg, epi, _, ex, inp = entry
        if name == "gather":
            gather(xin, segs)
        elif inp is not None and M <= 16:
            _lib.gemv_input(xin, segs, nseg, inp, epilogue=epi, flags=flags & ~(_lib.FLAG_TILE_KERNEL | _lib.FLAG_ROWS_KERNEL),
                            ex=ex)
        elif name == "fht":
            _lib.fht(xin, nseg, out=segs)       # (src, dst, signs) ride in the entry's slots
        elif ex is not None:
            # library policy: the flag array was sized with gemv_launch_blocks for the same policy
            _lib.gemv_exchange(xin, segs, nseg, ex, epilogue=epi, split=0, flags=flags & ~(_lib.FLAG_TILE_KERNEL | _lib.FLAG_ROWS_KERNEL))
        elif M <= 16:
            _lib.gemv_multi(xin, segs, nseg, epilogue=epi, flags=flags)
        elif epi == _lib.EPI_SILU_MUL:
            # prefill: gate and up as full-width tensor-core tiles of ONE launch, then one
            # SiLU*mul pass (measured faster than the fused 128-token form and than folding the
            # multiply into the second projection's epilogue)
            descs = entry[5]
            for i in range(0, nseg, 2):
                act = descs[i]["out"]
                ubuf = self._scratch(act.shape, act.dtype)
                pair = [dict(descs[i], ldo=act.stride(0)), dict(descs[i + 1], out=ubuf, ldo=ubuf.shape[1])]
                if self.merge_prefill and _lib.gemm_multi_ok(pair, xin.shape[1]):
                    _lib.gemm_multi(xin, _lib.make_segments(pair), 2, flags=flags)
                else:
                    _lib.gemm(xin, _pair(segs, i, _lib.EPI_NONE), flags=flags)
                    _lib.gemm(xin, _lib.make_segments([pair[1]]), flags=flags)
                _lib.silu_mul(act, ubuf)
        else:
            descs = entry[5]
            i = 0
            while i < nseg:      # merged launches of up to four projections that share x
                j = min(nseg, i + _lib.GEMM_MULTI_MAX) if self.merge_prefill else i + 1
                if j - i > 1 and _lib.gemm_multi_ok(descs[i:j], xin.shape[1]):
                    _lib.gemm_multi(xin, ctypes.cast(ctypes.byref(segs[i]), ctypes.POINTER(_lib.Segment)),
                                    j - i, flags=flags)
                else:
                    j = i + 1
                    _lib.gemm(xin, _pair(segs, i, epi), epilogue=epi, flags=flags)
                i = j

    def _scratch(self, shape, dtype) -> torch.Tensor:
        buf = self.__dict__.get("_scratch_buf")
        if buf is None or buf.shape != tuple(shape) or buf.dtype != dtype:
            buf = torch.empty(tuple(shape), dtype=dtype, device=self.device)
            self.__dict__["_scratch_buf"] = buf
        return buf

    def step(self, M: int, flags: int = 0, gather=None) -> torch.Tensor:
        """Run every projection once on the plan's activation buffer; returns the
        last layer's down_proj output (this rank's columns)."""
        plan = self._plan(M)
        for entry in plan["launches"]:
            self.run_launch(entry, M, flags, gather)
        return plan["y"]

    def check_status(self) -> None:
        """Call after a host sync (it reads a device word): raises when a bounded wait ran out in
        any kernel since the last call — a peer's push that never came (0x7000 + rank), a
        tensor-core pipeline wait, an embedding id out of range. From the first expiry until this
        call the step's outputs are undefined; after an exchange expiry re-zero the arenas
        (every rank) before the next step."""
        status = _lib.lib().b200lut_device_status()
        if status != 0:
            raise RuntimeError(f"LinearStack: a bounded device wait ran out (device status {status:#x})")

    def decode_plans(self, M: int):
        """Persistent-launch form of the step (M <= 16): the launches between two
        all-gathers become one plan each (a single plan on one GPU). Inside a plan every
        job depends on the one before it — the order a real decoder layer imposes."""
        plan = self._plan(M)
        if "plans" not in plan:
            groups, cur = [], []
            for name, xin, segs, nseg, epi, descs, _, inp in plan["launches"]:
                if name == "fht" or inp is not None:
                    raise ValueError("the persistent executor does not serve a rotated stack")
                if name == "gather":
                    groups.append(("plan", cur))
                    groups.append(("gather", (xin, segs)))
                    cur = []
                else:
                    cur.append(dict(x=xin, segs=descs, epilogue=epi, dep=len(cur) - 1))
            groups.append(("plan", cur))
            plan["plans"] = [(k, _lib.DecodePlan(v, M, self.dtype, self.device) if k == "plan" else v)
                             for k, v in groups if k == "gather" or v]
        return plan["plans"]

    def step_persistent(self, M: int, gather=None) -> torch.Tensor:
        for kind, item in self.decode_plans(M):
            if kind == "plan":
                item.run()
            else:
                gather(*item)
        return self._plan(M)["y"]

    def launches_per_step(self, M: int) -> int:
        """Kernel launches of one step (the all-gathers of a multi-GPU step not counted)."""
        n = 0
        for name, xin, _, nseg, epi, descs, _, _ in self._plan(M)["launches"]:
            if name == "gather":
                continue
            if M <= 16 or name == "fht":
                n += 1
                continue
            K = xin.shape[1]
            if epi == _lib.EPI_SILU_MUL:     # per pair: merged (1) or separate (2) GEMMs + SiLU*mul
                for i in range(0, nseg, 2):
                    merged = self.merge_prefill and _lib.gemm_multi_ok(descs[i:i + 2], K)
                    n += (1 if merged else 2) + 1
            else:
                i = 0
                while i < nseg:
                    j = min(nseg, i + _lib.GEMM_MULTI_MAX) if self.merge_prefill else i + 1
                    if not (j - i > 1 and _lib.gemm_multi_ok(descs[i:j], K)):
                        j = i + 1
                    n += 1
                    i = j
        return n


def _pair(segs, i, epi):
    """Pointer to segment i of a ctypes segment array (the prefill GEMM takes one
    projection, or one (gate, up) pair merged into a single descriptor)."""
    import ctypes
    if epi != _lib.EPI_SILU_MUL:
        return ctypes.pointer(segs[i])
    s = _lib.Segment()
    ctypes.memmove(ctypes.byref(s), ctypes.byref(segs[i]), ctypes.sizeof(s))
    s.packed2, s.lut2, s.bits2 = segs[i + 1].packed, segs[i + 1].lut, segs[i + 1].bits
    return ctypes.pointer(s)
