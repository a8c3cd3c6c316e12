"""Tensor-parallel linear on 2 GPUs (NCCL): every rank ends with the full output, equal to the
single-GPU result of the same kernels and inside the parity bar against the fp64 oracle.
Skipped when fewer than 2 GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import nanoquant_oracle as oc

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nanoquant_b200 import ops, tp
        from nanoquant_b200.kernel import utils as ku
        from tests.util import parity_excess, TOL, exact_np, half2_bits, make_layer
        out = []
        for (N, R, M, T) in ((1024, 288, 1024, 1), (2048, 512, 4096, 3), (1024, 256, 2048, 160)):
            L = make_layer(N, R, M, T, torch.bfloat16, seed=N + T, device=f"cuda:{rank}")
            vt = ku.pack_tiles(half2_bits(L["V"], f"cuda:{rank}"), (R, N), "half2")
            ut = ku.pack_tiles(half2_bits(L["U"], f"cuda:{rank}"), (M, R), "half2")
            shard = tp.TPLinearShard.from_full(vt, ut, L["s_pre"], L["s_mid"], L["s_post"], N, R, M, world, rank)
            y = tp.tp_linear_forward(L["x"], shard)
            y1 = ops.linear_forward(L["x"], L["s_pre"], vt, L["s_mid"], ut, L["s_post"], R)
            torch.cuda.synchronize()
            out.append((tuple(y.shape), bool(torch.equal(y, y1)), parity_excess(exact_np(y), L["y64"], torch.bfloat16) <= 0))
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


def test_tp_linear_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, out in results:
        for shape, same_as_single, in_bar in out:
            assert same_as_single and in_bar, (rank, shape)


def _peer_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nanoquant_b200 import tp
        dev = torch.device("cuda", rank)
        pg = tp.PeerGather(1 << 20)
        shapes = [((1, 512), torch.bfloat16), ((3, 2048), torch.float16), ((160, 1024), torch.bfloat16)]
        regions = [pg.region(sh, dt) for sh, dt in shapes]
        ok = []
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        # eager, twice over every region, then the same sequence replayed from a CUDA graph
        shards = [torch.randn(sh, generator=g, device=dev).to(dt) for sh, dt in shapes]
        for rep in range(2):
            for sh_t, reg in zip(shards, regions):
                sh_t.add_(1)                      # new data every round
                got = pg.gather(sh_t, reg)
                ref = [torch.empty_like(sh_t) for _ in range(world)]
                dist.all_gather(ref, sh_t)
                torch.cuda.synchronize()
                ok.append(bool(torch.equal(got, torch.stack(ref))))
        s = torch.cuda.Stream(dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            with torch.cuda.graph(graph, stream=s):
                for sh_t, reg in zip(shards, regions):
                    pg.gather(sh_t, reg)
        torch.cuda.current_stream(dev).wait_stream(s)
        for rep in range(3):
            for sh_t in shards:
                sh_t.mul_(2)
            graph.replay()
            torch.cuda.synchronize()
            for sh_t, reg in zip(shards, regions):
                ref = [torch.empty_like(sh_t) for _ in range(world)]
                dist.all_gather(ref, sh_t)
                torch.cuda.synchronize()
                ok.append(bool(torch.equal(reg, torch.stack(ref))))
        ok.append(pg.status() == 0)
        q.put((rank, ok))
    except Exception as e:   # report instead of leaving the parent waiting
        q.put((rank, [f"{type(e).__name__}: {e}"]))
    finally:
        dist.destroy_process_group()


def test_peer_memory_all_gather_two_gpus():
    """nq_allgather_push on symmetric memory against NCCL, eagerly and replayed from a CUDA graph."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok in results:
        assert all(v is True for v in ok), (rank, ok)
