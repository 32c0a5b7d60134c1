"""Partitioned matmul: the owner-computes plan and the K-chunked exchange schedule, on CPU ranks.

The multi-rank path runs as real torch.distributed processes over gloo with stand-in leaves
(a float64 matmul on the host plays the GPU), the way the reference tests its scheduler against
mock nodes that acknowledge work without a GPU (phobos-sched/src/server.rs:843-1039)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def part(ph):
    return sys.modules[ph.__name__ + ".partition"]


def test_grids_and_ownership(part):
    for world, (pr, pc) in {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}.items():
        plan = part.plan_partition(16384, 16384, 16384, world)
        assert (plan.pr, plan.pc) == (pr, pc)
        seen = np.zeros((pr, pc), dtype=int)
        for rank in range(world):
            r0, mb, c0, nb = plan.c_block(rank)
            assert (mb, nb) == (16384 // pr, 16384 // pc)
            seen[r0 // mb, c0 // nb] += 1
            assert plan.rank_of(*plan.coords(rank)) == rank
            assert rank in plan.row_group(rank) and rank in plan.col_group(rank)
        assert (seen == 1).all()                     # every C block has exactly one owner


def test_every_input_element_has_one_home(part):
    plan = part.plan_partition(512, 512, 1024, 8)
    a_cover = np.zeros((plan.pr, 1024), dtype=int)
    b_cover = np.zeros((plan.pc, 1024), dtype=int)
    for rank in range(8):
        r, c = plan.coords(rank)
        k0, w = plan.a_shard_k(rank)
        a_cover[r, k0:k0 + w] += 1
        k0, h = plan.b_shard_k(rank)
        b_cover[c, k0:k0 + h] += 1
    assert (a_cover == 1).all() and (b_cover == 1).all()


def test_steps_cover_k_once_and_point_at_their_homes(part):
    plan = part.plan_partition(1024, 1024, 4096, 8, k_chunk=256)
    assert [s.k0 for s in plan.steps] == list(range(0, 4096, 256))
    for s in plan.steps:
        assert s.a_home_col == s.k0 // (4096 // plan.pc)
        assert s.b_home_row == s.k0 // (4096 // plan.pr)
        assert s.a_local_chunk * 256 == s.k0 % (4096 // plan.pc)
        assert s.b_local_row0 == s.k0 % (4096 // plan.pr)
    with pytest.raises(ValueError):
        part.plan_partition(1024, 1024, 4096, 8, k_chunk=768)
    with pytest.raises(ValueError):
        part.plan_partition(1000, 1024, 4096, 3)


def test_peer_bytes_are_the_analytic_minimum(part):
    """Each rank must receive exactly the part of its A row-panel and B column-panel it is not home to
    (the reference pins fetch bytes to the analytic minimum, phobos-sched/src/lib.rs:1184-1185)."""
    M = N = K = 16384
    for world in (1, 2, 4, 8):
        plan = part.plan_partition(M, N, K, world)
        want = sum((M // plan.pr) * K * (plan.pc - 1) // plan.pc + (N // plan.pc) * K * (plan.pr - 1) // plan.pr
                   for _ in range(world)) * 4
        assert plan.total_peer_bytes() == want
    assert part.plan_partition(M, N, K, 1).total_peer_bytes() == 0
    assert part.plan_partition(M, N, K, 8).recv_bytes(0) == (8192 * 12288 + 4096 * 8192) * 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, kc, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    ph = entry.load_package()
    part = sys.modules[ph.__name__ + ".partition"]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = part.plan_partition(M, N, K, world, k_chunk=kc)
        A = torch.from_numpy(ph.fill_random_host(M * K, 1).reshape(M, K)).double()
        B = torch.from_numpy(ph.fill_random_host(K * N, 2).reshape(K, N)).double()
        C = torch.from_numpy(ph.fill_random_host(M * N, 3).reshape(M, N)).double()
        a_shard, b_shard, c_block = part.shard_inputs(plan, rank, A, B, C)
        row_pg, col_pg = part.make_groups(plan, rank)
        calls = {"init": 0, "step": 0}

        def leaf_init(Cb, beta):          # stand-in for the `matmul_init` leaf
            calls["init"] += 1
            Cb.mul_(beta)

        def leaf_step(Ak, Bk, Cb, alpha):  # stand-in for the `matmul` step leaf (beta = 1)
            calls["step"] += 1
            Cb.add_(alpha * (Ak @ Bk))

        part.run_partitioned(plan, rank, a_shard, b_shard, c_block, 0.125, 1.5, leaf_init, leaf_step, row_pg, col_pg)
        want = 0.125 * (A @ B) + 1.5 * C
        r0, mb, c0, nb = plan.c_block(rank)
        err = float((c_block - want[r0:r0 + mb, c0:c0 + nb]).abs().max())
        q.put((rank, err, calls["init"], calls["step"], len(plan.steps)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape,kc", [(2, (64, 96, 128), 32), (4, (64, 64, 96), 16), (8, (32, 64, 128), 16)])
def test_partitioned_schedule_on_gloo_ranks(world, shape, kc):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, *shape, kc, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    res = sorted(q.get(timeout=10) for _ in range(world))
    assert [r[0] for r in res] == list(range(world))
    for rank, err, n_init, n_step, n_plan in res:
        assert err < 1e-12, f"rank {rank}: {err}"
        assert n_init == 1 and n_step == n_plan       # one init leaf, one step leaf per K chunk
