"""Host logic of the output-dimension tensor-parallel split (two gloo ranks on CPU).  The local
shard is computed by the numpy oracle here; the point is the sharding and gathering arithmetic."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nanoquant_oracle as oc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nanoquant_b200 import tp
        N, R, M = 96, 64, 128
        d = oc.synth_linear(N, R, M, T, seed=3)
        lo, hi = tp.shard_bounds(M, world, rank)
        u_rows = tp.shard_rows_packed(torch.from_numpy(oc.pack_rows(d["U"], "lsb_first")), M, world, rank)
        assert u_rows.shape[0] == hi - lo
        U_local = oc.unpack_rows(u_rows.numpy(), (hi - lo, R), "lsb_first")
        shard = tp.TPLinearShard(None, None, None, None, None, N, R, M, world, rank)

        def local_fn(x, sh):
            y = oc.forward_fp64(x.numpy(), d["V"], U_local, d["s_pre"], d["s_mid"], d["s_post"][lo:hi])
            return torch.from_numpy(y)

        y = tp.tp_linear_forward(torch.from_numpy(d["x"].astype(np.float64)), shard, local_fn=local_fn)
        y64 = oc.forward_fp64(d["x"], d["V"], d["U"], d["s_pre"], d["s_mid"], d["s_post"])
        q.put((rank, tuple(y.shape), float(np.max(np.abs(y.numpy() - y64)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [1, 5])
def test_tp_shard_and_gather_two_ranks(T):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, shape, err in results:
        assert shape == (T, 128)
        assert err == 0.0   # the gathered result is exactly the unsharded oracle on every rank


def test_shard_bounds_and_tile_views():
    from nanoquant_b200 import tp
    assert tp.shard_bounds(4096, 8, 3) == (1536, 2048)
    with pytest.raises(ValueError):
        tp.shard_bounds(1000, 8, 0)
    tiles = torch.arange(64 * 3 * 128, dtype=torch.int32).view(64, 3, 128)    # 1024 rows
    s = tp.shard_rows_tiles(tiles, 1024, 4, 2)
    assert s.shape == (16, 3, 128) and torch.equal(s, tiles[32:48])
