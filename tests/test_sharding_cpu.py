"""Column-parallel sharding on CPU ranks (gloo, world size 2 and 4): every rank takes its
slice of the idxN blob and of the palette rows, computes its output columns with the oracle,
and the all-gathered result must equal the unsharded forward bit for bit (same per-row
arithmetic). Covers the host-side shard logic the GPU stack uses."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_NAME, ROOT


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, M: int, ret):
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        st = importlib.import_module(PKG_NAME + ".stack")
        syn = importlib.import_module(PKG_NAME + ".synthetic")
        from oracle import lut_linear_oracle as orc
        N, K, bits, gs = 1024, 256, 4, 128
        codes, blob = syn.make_blob(N, K, bits, 11)
        lut = syn.make_lut(N // gs, bits, torch.bfloat16, 11)
        x = syn.make_x(M, K, torch.bfloat16, 12)
        full = orc.linear_forward(x, orc.dequant(blob.numpy(), lut, N, K, gs, bits))
        n_loc = N // world
        my_blob = st.shard_blob(blob, N, K, bits, rank, world)
        my_lut = st.shard_lut(lut, N, gs, rank, world)
        assert np.array_equal(orc.unpack_idxn(my_blob.numpy(), n_loc, K, bits),
                              codes[rank * n_loc:(rank + 1) * n_loc])
        mine = orc.linear_forward(x, orc.dequant(my_blob.numpy(), my_lut, n_loc, K, gs, bits))
        # the gather used by the stack: rank-major pieces, then a permute for M > 1
        tmp = torch.empty(world, M, n_loc, dtype=torch.float32)
        dist.all_gather_into_tensor(tmp.view(-1), mine.float().contiguous().view(-1))
        got = tmp.permute(1, 0, 2).reshape(M, N)
        ret[rank] = bool(torch.equal(got, full.float()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,M", ((2, 1), (2, 8), (4, 3)))
def test_sharded_forward_equals_unsharded(world, M):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world))


def test_shard_refusals():
    import importlib
    st = importlib.import_module(PKG_NAME + ".stack")
    with pytest.raises(ValueError):
        st.shard_rows(1024, 128, 0, 3)
    assert st.shard_rows(1024, 128, 3, 8) == (384, 512)
    assert st.census() == {"modules": 248, "weights": 6912212992}
