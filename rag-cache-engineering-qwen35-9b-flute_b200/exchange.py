"""Peer-mapped exchange buffers for the column-parallel decode stack.

The reference runs on one GPU and has no counterpart of this module. Here every rank
(one process per GPU of one box) owns a zero-filled device buffer — its arena — that
all other ranks map through CUDA IPC. A producing GEMV stores its output slice into its
own arena and, over NVLink, into the same place of every peer's arena, then raises a
flag word there; the consuming GEMV waits for the flags (see `b200lut_exchange` in
include/b200_lut.h). No collective call and no extra launch sits between the two.

All ranks must carve their arenas with the same sequence of `alloc` calls, so that an
offset names the same slot everywhere.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _lib

_ALIGN = 256


class PeerArena:
    """`nbytes` of zeroed device memory per rank, addressable from every rank."""

    def __init__(self, nbytes: int, rank: int, world: int, device, group=None):
        import torch.distributed as dist
        self.rank, self.world = rank, world
        self.nbytes = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        mine = _lib.peer_export(self.buf)
        everyone: List[Optional[tuple]] = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        self._opened = []
        self.base = []
        for r, (handle, off) in enumerate(everyone):
            if r == rank:
                self.base.append(self.buf.data_ptr())
            else:
                with torch.cuda.device(device):
                    b = _lib.peer_open(handle)
                self._opened.append(b)
                self.base.append(b + off)
        self._cursor = 0
        self.emulated = False
        self._group = group
        dist.barrier(group=group)      # every rank has zeroed and mapped before anyone pushes

    @classmethod
    def emulated(cls, nbytes: int, world: int, device) -> List["PeerArena"]:
        """`world` arenas on ONE device (each "rank" sees the others by plain pointers):
        the single-GPU test form, driven by launches issued one after the other."""
        arenas = []
        nbytes = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        for r in range(world):
            a = cls.__new__(cls)
            a.rank, a.world, a.nbytes, a.buf = r, world, nbytes, bufs[r]
            a._opened, a._cursor = [], 0
            a.emulated, a._group = True, None
            a.base = [b.data_ptr() for b in bufs]
            arenas.append(a)
        return arenas

    def alloc(self, nbytes: int) -> int:
        """Offset of a fresh 256-byte-aligned slot."""
        off = self._cursor
        self._cursor = off + (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        if self._cursor > self.nbytes:
            raise ValueError(f"arena of {self.nbytes} bytes is full")
        return off

    def view(self, off: int, shape, dtype) -> torch.Tensor:
        """Tensor over the local arena at `off`."""
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buf[off:off + nbytes].view(dtype).view(*shape)

    def ready(self, device) -> None:
        """After channels have been carved and pre-filled: every rank's fills have landed before
        any rank pushes (nothing to do for arenas emulated on one device, whose launches are
        issued in order)."""
        if self.emulated:
            return
        import torch.distributed as dist
        torch.cuda.synchronize(device)
        dist.barrier(group=self._group)

    def close(self) -> None:
        for b in self._opened:
            _lib.peer_close(b)
        self._opened = []


class Channel:
    """One exchanged activation buffer [M, width] with its flag array and counters. `blocks` is
    the block count of the producing launch (`_lib.gemv_launch_blocks` of its segments): every
    block of it owns one flag. sentinel=True: no flags — the buffer starts filled with 0xFFFF, the
    consumer polls the rows themselves and refills them after use (row-range kernel only; the
    caller synchronises the ranks once after building its channels, before the first push)."""

    def __init__(self, arena: PeerArena, M: int, width: int, dtype, blocks: int, sentinel: bool = False):
        self.arena = arena
        self.blocks = int(blocks)
        self.act_off = arena.alloc(M * width * 2)
        self.flag_off = arena.alloc(arena.world * self.blocks * 4)
        # local counters: push ticket +0, push count +32, wait ticket +64, wait count +96
        self.ctl_off = arena.alloc(_ALIGN)
        self.act = arena.view(self.act_off, (M, width), dtype)
        self.sentinel = bool(sentinel)
        if self.sentinel:
            arena.buf[self.act_off:self.act_off + M * width * 2].fill_(0xFF)
        a = arena
        me = a.base[a.rank]
        push = _lib.Exchange()
        push.world, push.rank, push.push, push.wait = a.world, a.rank, 1, 0
        push.producer_blocks = self.blocks
        for q in range(a.world):
            push.peer_delta[q] = a.base[q] - me
            push.peer_flag[q] = a.base[q] + self.flag_off
        push.ticket = me + self.ctl_off
        push.epoch = me + self.ctl_off + 32
        wait = _lib.Exchange()
        wait.world, wait.rank, wait.push, wait.wait = a.world, a.rank, 0, 1
        wait.producer_blocks = self.blocks
        wait.flags = me + self.flag_off
        wait.wait_ticket = me + self.ctl_off + 64
        wait.wait_count = me + self.ctl_off + 96
        push.sentinel = wait.sentinel = 1 if self.sentinel else 0
        self.push, self.wait = push, wait
