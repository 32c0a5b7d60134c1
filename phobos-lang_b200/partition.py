"""Partitioned `matmul` over the GPUs of one box: the cluster path for one kernel.

The reference plans a `@cluster` matmul as independent C supertiles, each owned by
one node (`lin % nodes`, phobos-sched/src/lib.rs:591-600), computed as one init
leaf `C = beta*C` followed by a chain of step leaves `C = alpha*(A_k @ B_k) + C`
over the K supertiles (phobos-cluster/src/clustergen.rs:94-120, 1276-1399); input
supertiles are LOADed by their lowest-id consumer and FETCHed by the others over
gRPC (`HomeLoadPeerFetch`, phobos-sched/src/lib.rs:17-25, 615-620, 691-713).

Here the same algebra runs on a pr x pc grid of ranks, one process per GPU:
rank (r, c) owns the C block [M/pr, N/pc].  The A row-panel r starts split over
the pc ranks of grid row r (by K), the B column-panel c over the pr ranks of grid
column c (by K) — each input element has exactly one home, as in the reference.
K is walked in chunks; the A chunk of a step is broadcast inside the grid row by
its home rank and the B chunk inside the grid column (NCCL over NVLink, landing
in local HBM), on a side stream one step ahead of the step leaf that consumes
it.  No kernel reads peer memory.

`plan_partition` is pure host logic.  `run_partitioned` drives the exchange with
torch.distributed and calls the leaves through callables, so the schedule can be
exercised on CPU ranks (gloo) with stand-in leaves, the way the reference tests
its scheduler against mock nodes (phobos-sched/src/server.rs:843-1039).
"""
from __future__ import annotations

from dataclasses import dataclass
from math import gcd

GRIDS = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}


@dataclass(frozen=True)
class Step:
    """One step leaf: C += alpha * A[:, k0:k0+kc] @ B[k0:k0+kc, :] on every rank."""
    index: int
    k0: int
    kc: int
    a_home_col: int      # grid column whose ranks hold this A chunk
    a_local_chunk: int   # chunk index inside the home rank's A shard
    b_home_row: int      # grid row whose ranks hold this B chunk
    b_local_row0: int    # first row of the chunk inside the home rank's B shard


@dataclass(frozen=True)
class PartitionPlan:
    M: int
    N: int
    K: int
    world: int
    pr: int
    pc: int
    kc: int
    steps: tuple

    # ---- ownership -------------------------------------------------------------
    def coords(self, rank: int) -> tuple:
        return rank // self.pc, rank % self.pc

    def rank_of(self, r: int, c: int) -> int:
        return r * self.pc + c

    @property
    def mb(self) -> int:
        return self.M // self.pr

    @property
    def nb(self) -> int:
        return self.N // self.pc

    def c_block(self, rank: int) -> tuple:
        """(row0, rows, col0, cols) of the C block the rank owns."""
        r, c = self.coords(rank)
        return r * self.mb, self.mb, c * self.nb, self.nb

    def a_shard_k(self, rank: int) -> tuple:
        """(k0, k_extent) of the A row-panel slice whose home is this rank."""
        _, c = self.coords(rank)
        w = self.K // self.pc
        return c * w, w

    def b_shard_k(self, rank: int) -> tuple:
        """(k0, k_extent) of the B column-panel slice whose home is this rank."""
        r, _ = self.coords(rank)
        h = self.K // self.pr
        return r * h, h

    def row_group(self, rank: int) -> list:
        r, _ = self.coords(rank)
        return [self.rank_of(r, c) for c in range(self.pc)]

    def col_group(self, rank: int) -> list:
        _, c = self.coords(rank)
        return [self.rank_of(r, c) for r in range(self.pr)]

    # ---- traffic ------------------------------------------------------------------
    def recv_bytes(self, rank: int, elem_bytes: int = 4) -> int:
        """Bytes a rank receives: its A panel and B panel minus what it is home to."""
        a = self.mb * (self.K - self.K // self.pc)
        b = self.nb * (self.K - self.K // self.pr)
        return (a + b) * elem_bytes

    def total_peer_bytes(self, elem_bytes: int = 4) -> int:
        return sum(self.recv_bytes(rk, elem_bytes) for rk in range(self.world))


def plan_partition(M: int, N: int, K: int, world: int, k_chunk: int | None = None) -> PartitionPlan:
    """2-D owner-computes plan for `world` ranks (1, 2, 4 or 8)."""
    if world not in GRIDS:
        raise ValueError(f"world size {world} not in {sorted(GRIDS)}")
    pr, pc = GRIDS[world]
    if M % pr or N % pc or K % pr or K % pc:
        raise ValueError(f"M, N, K = {M}, {N}, {K} do not divide over a {pr}x{pc} grid")
    wa, hb = K // pc, K // pr          # home slice extents along K
    base = gcd(wa, hb)                 # finest common refinement of both slicings
    kc = base if k_chunk is None else k_chunk
    if base % kc:
        raise ValueError(f"k_chunk {kc} does not divide the common K slice {base}")
    steps = []
    for i, k0 in enumerate(range(0, K, kc)):
        steps.append(Step(index=i, k0=k0, kc=kc, a_home_col=k0 // wa, a_local_chunk=(k0 % wa) // kc,
                          b_home_row=k0 // hb, b_local_row0=k0 % hb))
    return PartitionPlan(M=M, N=N, K=K, world=world, pr=pr, pc=pc, kc=kc, steps=tuple(steps))


def default_k_chunk(plan_K: int, world: int, target: int = 2048) -> int:
    """Largest chunk <= target that divides the common K slice."""
    pr, pc = GRIDS[world]
    base = gcd(plan_K // pc, plan_K // pr)
    kc = min(base, target)
    while base % kc:
        kc -= 1
    return kc


def shard_inputs(plan: PartitionPlan, rank: int, A, B, C):
    """Cuts a rank's home shards out of full A, B, C tensors (torch, any device).

    Returns (a_shard [chunks, mb, kc], b_shard [K/pr, nb], c_block [mb, nb]); the A
    shard is stored chunk-major so that every exchanged chunk is contiguous.
    """
    r, c = plan.coords(rank)
    row0, mb, col0, nb = plan.c_block(rank)
    ak0, aw = plan.a_shard_k(rank)
    bk0, bh = plan.b_shard_k(rank)
    a = A[row0:row0 + mb, ak0:ak0 + aw]
    a_shard = a.reshape(mb, aw // plan.kc, plan.kc).permute(1, 0, 2).contiguous()
    b_shard = B[bk0:bk0 + bh, col0:col0 + nb].contiguous()
    c_block = C[row0:row0 + mb, col0:col0 + nb].contiguous()
    return a_shard, b_shard, c_block


def run_partitioned(plan: PartitionPlan, rank: int, a_shard, b_shard, c_block, alpha: float, beta: float,
                    leaf_init, leaf_step, row_pg=None, col_pg=None, comm_stream=None, compute_stream=None,
                    buffers=None, peers=None):
    """Runs init + the chain of step leaves on this rank; c_block is updated in place.

    leaf_init(C, beta) and leaf_step(A_chunk, B_chunk, C, alpha) are the leaves
    (`matmul_init`, and `matmul` with beta = 1).  row_pg / col_pg are the process
    groups of the rank's grid row / column (None when the group has one member).
    With CUDA tensors the broadcasts of step t+1 run on `comm_stream` while the
    leaf of step t runs on `compute_stream`.  With `peers` (a PeerShards) there is no
    collective at all: every rank copies the chunks it is not home to straight out of the
    home rank's shard (device-to-device copies over NVLink on `comm_stream`), and a_shard /
    b_shard must be the tensors PeerShards holds.
    """
    import torch
    import torch.distributed as dist

    r, c = plan.coords(rank)
    cuda = c_block.is_cuda
    if buffers is None:
        buffers = alloc_buffers(plan, a_shard, b_shard)
    a_buf, b_buf = buffers
    n = len(plan.steps)
    ready = [None] * n      # event: chunk data of step i is in local memory
    consumed = [None] * n   # event: leaf of step i has finished reading its buffers
    a_use, b_use = [None] * n, [None] * n

    def stage(i: int) -> None:
        st = plan.steps[i]
        a_local = st.a_home_col == c
        b_local = st.b_home_row == r
        a_src = a_shard[st.a_local_chunk] if a_local else None
        b_src = b_shard[st.b_local_row0:st.b_local_row0 + st.kc] if b_local else None
        ctx = torch.cuda.stream(comm_stream) if cuda and comm_stream is not None else _Null()
        with ctx:
            if cuda and i >= 2 and consumed[i - 2] is not None:
                comm_stream.wait_event(consumed[i - 2])   # buffer (i % 2) is free again
            if peers is not None:
                if plan.pc > 1 and not a_local:
                    a_src = a_buf[i % 2]
                    a_src.copy_(peers.a_chunk(plan.rank_of(r, st.a_home_col), st.a_local_chunk), non_blocking=True)
                if plan.pr > 1 and not b_local:
                    b_src = b_buf[i % 2]
                    b_src.copy_(peers.b_rows(plan.rank_of(st.b_home_row, c), st.b_local_row0, st.kc), non_blocking=True)
            elif plan.pc > 1:
                if a_local:
                    dist.broadcast(a_src, src=plan.rank_of(r, st.a_home_col), group=row_pg)
                else:
                    a_src = a_buf[i % 2]
                    dist.broadcast(a_src, src=plan.rank_of(r, st.a_home_col), group=row_pg)
            if peers is None and plan.pr > 1:
                if b_local:
                    dist.broadcast(b_src, src=plan.rank_of(st.b_home_row, c), group=col_pg)
                else:
                    b_src = b_buf[i % 2]
                    dist.broadcast(b_src, src=plan.rank_of(st.b_home_row, c), group=col_pg)
            if cuda and comm_stream is not None:
                ev = torch.cuda.Event()
                ev.record(comm_stream)
                ready[i] = ev
        a_use[i], b_use[i] = a_src, b_src

    cctx = torch.cuda.stream(compute_stream) if cuda and compute_stream is not None else _Null()
    if cuda:
        # whatever the caller queued on its current stream (filling or restoring the shards and C)
        # comes before anything this run does on its own streams
        here = torch.cuda.current_stream()
        if compute_stream is not None:
            compute_stream.wait_stream(here)
        if comm_stream is not None:
            comm_stream.wait_stream(here)
    if cuda and comm_stream is not None and compute_stream is not None:
        comm_stream.wait_stream(compute_stream)
    stage(0)
    with cctx:
        leaf_init(c_block, beta)
    for i in range(n):
        if i + 1 < n:
            stage(i + 1)
        with cctx:
            if cuda and ready[i] is not None:
                (compute_stream or torch.cuda.current_stream()).wait_event(ready[i])
            leaf_step(a_use[i], b_use[i], c_block, alpha)
            if cuda and compute_stream is not None:
                ev = torch.cuda.Event()
                ev.record(compute_stream)
                consumed[i] = ev
    return c_block


class PeerShards:
    """The home shards of all ranks, readable from every rank of the box.

    Each rank puts its A and B home shards into symmetric memory (same shape on every rank, mapped into
    every process over NVLink); `a_chunk` / `b_rows` return a view of another rank's shard that a plain
    device-to-device copy can read.  The shards are inputs and never change during a run, so readers
    need no handshake beyond the one barrier after they are filled.
    """

    def __init__(self, plan: PartitionPlan, rank: int, a_shard, b_shard):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.plan = plan
        self.a_shape, self.b_shape = tuple(a_shard.shape), tuple(b_shard.shape)
        self.dtype = a_shard.dtype
        self.a = symm.empty(self.a_shape, dtype=a_shard.dtype, device=a_shard.device)
        self.b = symm.empty(self.b_shape, dtype=b_shard.dtype, device=b_shard.device)
        self.a.copy_(a_shard)
        self.b.copy_(b_shard)
        self._ha = symm.rendezvous(self.a, dist.group.WORLD)
        self._hb = symm.rendezvous(self.b, dist.group.WORLD)
        self._views = {}
        import torch
        torch.cuda.synchronize()
        dist.barrier()                 # every shard is filled before anyone reads one

    def _peer(self, which: str, peer_rank: int):
        key = (which, peer_rank)
        if key not in self._views:
            h, shape = (self._ha, self.a_shape) if which == "a" else (self._hb, self.b_shape)
            self._views[key] = h.get_buffer(peer_rank, shape, self.dtype)
        return self._views[key]

    def a_chunk(self, peer_rank: int, chunk: int):
        return self._peer("a", peer_rank)[chunk]

    def b_rows(self, peer_rank: int, row0: int, rows: int):
        return self._peer("b", peer_rank)[row0:row0 + rows]


def alloc_buffers(plan: PartitionPlan, a_shard, b_shard):
    """Two receive buffers per operand (the chunk in use and the chunk in flight)."""
    import torch
    a_buf = [torch.empty((plan.mb, plan.kc), dtype=a_shard.dtype, device=a_shard.device) for _ in range(2)]
    b_buf = [torch.empty((plan.kc, plan.nb), dtype=b_shard.dtype, device=b_shard.device) for _ in range(2)]
    return a_buf, b_buf


def make_groups(plan: PartitionPlan, rank: int, max_ctas: int = 0):
    """Creates the row and column process groups (collective: every rank calls it).

    `max_ctas` > 0 (or PHOBOS_NCCL_MAX_CTAS) limits the NCCL groups to that many thread blocks, so that the
    exchange occupies fewer SMs next to the step leaf.  Measured at 16384^3: on 2 GPUs (one 128 MiB A chunk
    per step) 98.0 TFLOP/s with 4-8 blocks against 95.0 with NCCL's own choice, but on 4 GPUs (two 64 MiB
    chunks per step) 186 with 8 and 174 with 4 against 191: the default stays NCCL's own choice.
    """
    import torch.distributed as dist

    import os
    max_ctas = int(os.environ.get("PHOBOS_NCCL_MAX_CTAS", max_ctas))   # 0: NCCL's own choice

    def new_group(ranks):
        if dist.get_backend() == "nccl" and max_ctas > 0:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = max_ctas
            opts.config.min_ctas = 1
            return dist.new_group(ranks, pg_options=opts)
        return dist.new_group(ranks)

    row_pg = col_pg = None
    for r in range(plan.pr):
        ranks = [plan.rank_of(r, c) for c in range(plan.pc)]
        g = new_group(ranks) if len(ranks) > 1 else None
        if rank in ranks:
            row_pg = g
    for c in range(plan.pc):
        ranks = [plan.rank_of(r, c) for r in range(plan.pr)]
        g = new_group(ranks) if len(ranks) > 1 else None
        if rank in ranks:
            col_pg = g
    return row_pg, col_pg


def cuda_leaves():
    """The native leaves: `matmul_init` and `matmul` (beta = 1) through the C ABI.  The step leaf owns one
    workspace that grows to the largest step it has seen (the steps of a rank run one after another on the
    compute stream, so they may share it); with it the FFMA kernel reads a transposed copy of the A block."""
    import torch

    from . import F32, GEMM_FP32, gemm, gemm_workspace_bytes, matmul_init

    state = {"ws": None}

    def leaf_init(C, beta):
        matmul_init(C, beta)

    def leaf_step(A, B, C, alpha):
        need = gemm_workspace_bytes(GEMM_FP32, F32, A.shape[0], B.shape[1], A.shape[1])
        ws = state["ws"]
        if need and (ws is None or ws.numel() < need or ws.device != A.device):
            ws = state["ws"] = torch.empty((need,), dtype=torch.uint8, device=A.device)
        gemm(A, B, C, alpha, 1.0, GEMM_FP32, workspace=ws if need else None)

    return leaf_init, leaf_step


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
