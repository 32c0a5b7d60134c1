"""Partitioned matmul on real GPUs, one process per GPU over NCCL: both exchange forms against the oracle.
Needs at least two GPUs in the box (skipped otherwise)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, kc, exchange, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    ph = entry.load_package()
    part = sys.modules[ph.__name__ + ".partition"]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        plan = part.plan_partition(M, N, K, world, k_chunk=kc)
        A = torch.from_numpy(ph.fill_random_host(M * K, 1).reshape(M, K))
        B = torch.from_numpy(ph.fill_random_host(K * N, 2).reshape(K, N))
        C = torch.from_numpy(ph.fill_random_host(M * N, 3).reshape(M, N))
        a_shard, b_shard, c_block = (t.to(dev) for t in part.shard_inputs(plan, rank, A, B, C))
        row_pg, col_pg = part.make_groups(plan, rank)
        leaf_init, leaf_step = part.cuda_leaves()
        peers = part.PeerShards(plan, rank, a_shard, b_shard) if exchange == "p2p" else None
        pa, pb = (peers.a, peers.b) if peers is not None else (a_shard, b_shard)
        comm, comp = torch.cuda.Stream(), torch.cuda.Stream()
        for _ in range(2):                      # twice: the second run reuses buffers and events
            cb = c_block.clone()
            part.run_partitioned(plan, rank, pa, pb, cb, 0.125, 1.5, leaf_init, leaf_step, row_pg, col_pg,
                                 comm_stream=comm, compute_stream=comp, peers=peers)
            torch.cuda.synchronize()
        ph.device_status()
        r0, mb, c0, nb = plan.c_block(rank)
        q.put((rank, r0, mb, c0, nb, cb.cpu().numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "nccl"])
def test_partitioned_matmul_on_gpus(oracle, exchange):
    import torch
    import torch.multiprocessing as mp
    ndev = torch.cuda.device_count()
    if ndev < 2:
        pytest.skip("needs two GPUs")
    world = 8 if ndev >= 8 else 4 if ndev >= 4 else 2
    M, N, K, kc = 1024, 1024, 2048, 256
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, kc, exchange, q)) for r in range(world)]
    for p in procs:
        p.start()
    blocks = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    want = oracle.gemm_rows(a, b, c, 0.125, 1.5).reshape(M, N)
    got = np.zeros((M, N), np.float32)
    for rank, r0, mb, c0, nb, blk in blocks:
        got[r0:r0 + mb, c0:c0 + nb] = blk
    assert oracle.rel_frobenius(got, want) <= 1e-5
