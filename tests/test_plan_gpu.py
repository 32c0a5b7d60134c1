"""Job file -> kernel declaration -> supertile plan -> executors, on a B200 (one or two nodes of one box)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GEMM_PH = """
@cluster(SM in [256, 1024], SN in [256, 1024], SK in [256, 1024])
@autotune(SM in [32, 256], SN in [32, 256], SK in [4, 32])
kernel gemm(A: tensor<f32>[M, K], B: tensor<f32>[K, N], C: tensor<f32>[M, N], alpha: f32, beta: f32) {
  let i = program_id(0)
  let j = program_id(1)
  var acc: tile<f32>[SM, SN] = 0.0
  for k0 in range(0, K, SK) {
    acc += dot(A[i * SM :+ SM, k0 :+ SK], B[k0 :+ SK, j * SN :+ SN])
  }
  let before = C[i * SM :+ SM, j * SN :+ SN]
  C[i * SM :+ SM, j * SN :+ SN] = alpha * acc + beta * before
}
"""

FLASH_PH = """
@cluster(ROWS in [512, 2048])
@tensorcore
@launch(128)
@autotune(D in [128], ROWS in [4, 128], COLS in [4, 128])
kernel flash_attention(Q: tensor<f16>[Nq, D], K: tensor<f16>[Nk, D], V: tensor<f16>[Nk, D], O: tensor<f16>[Nq, D],
                       scale: f32) {
  let first = program_id(0) * ROWS
  let q = Q[first :+ ROWS, :]
  var acc: tile<f32>[ROWS, D] = 0.0
  var top: tile<f32>[ROWS, 1] = -65504.0
  var den: tile<f32>[ROWS, 1] = 0.0
  for c0 in range(0, Nk, COLS) {
    var s: tile<f32>[ROWS, COLS] = dot_t(q, K[c0 :+ COLS, :])
    s = s * scale
    var now: tile<f32>[ROWS, 1] = tmax(top, rowmax(s))
    s = exp(s - now)
    var fix: tile<f32>[ROWS, 1] = exp(top - now)
    den = den * fix
    den += rowsum(s)
    acc = acc * fix
    acc += dot(s, V[c0 :+ COLS, :])
    top = now
  }
  acc = acc / den
  O[first :+ ROWS, :] = acc
}
"""


def _tensors(job):
    return [(t.uri, t.dtype, t.shape, t.mode) for t in job.tensors]


@pytest.mark.parametrize("nodes,policy", [(1, "direct"), (2, "direct"), (2, "fetch")])
def test_gemm_job_planned_and_executed(ph, oracle, dev, tmp_path, nodes, policy):
    """`C = alpha*A@B + beta*C` from a job file: beta once by the init leaf, then K/SK accumulate steps per
    C supertile (which all carry the job's beta and must ignore it), outputs stored by their owners."""
    import torch
    M, N, K = 1024, 512, 768
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    for name, x in zip("abc", (a, b, c)):
        ph.store_region(f"file://{tmp_path}/{name}.tensor", x.shape, (0, 0), x)
    (tmp_path / "gemm.ph").write_text(GEMM_PH)
    (tmp_path / "job.txt").write_text(f"""
# C = 0.125 * A @ B + 1.5 * C
source = {tmp_path}/gemm.ph
dim M = {M}
dim N = {N}
dim K = {K}
tensor A = read f32 {M}x{K} file://{tmp_path}/a.tensor
tensor B = read f32 {K}x{N} file://{tmp_path}/b.tensor
tensor C = rmw  f32 {M}x{N} file://{tmp_path}/c.tensor
scalar alpha = f32 0.125
scalar beta = f32 1.5
""")
    job = ph.parse_job(str(tmp_path / "job.txt"))
    prog = ph.Program(job.source)
    assert prog.name == job.kernel == "gemm"
    prog.check_job(job)
    scalars = {s.name: ph.PhScalar(0, s.dtype, s.bits) for s in job.scalars}
    pl = ph.plan(prog, job.dims, nodes=nodes, scalars=scalars,
                 policy=ph.HOME_LOAD_PEER_FETCH if policy == "fetch" else ph.DIRECT_LOAD)
    pl.validate()
    assert len(pl.stores) == (M // 256) * (N // 256)
    if policy == "fetch":
        assert pl.fetch_bytes > 0
    ndev = torch.cuda.device_count()
    exs = [ph.Executor(n if n < ndev else 0, n, 16 << 20) for n in range(nodes)]
    try:
        ph.run_plan(pl, prog, _tensors(job), exs)
        for n, ex in enumerate(exs):
            done = ex.completions()
            assert sorted(d[0] for d in done) == sorted(i.iid for i in pl.node_instrs(n))
            assert all(d[1] == 0 for d in done) and ex.arena_used == 0
        if policy == "fetch":
            assert sum(ex.served_bytes for ex in exs) == pl.fetch_bytes
    finally:
        for ex in exs:
            ex.close()
    got = ph.load_region(f"file://{tmp_path}/c.tensor", (M, N), (0, 0), (M, N))
    assert oracle.rel_frobenius(got, oracle.gemm_rows(a, b, c, 0.125, 1.5)) <= 1e-5


@pytest.mark.parametrize("nodes,policy", [(1, "direct"), (2, "fetch"), (4, "fetch")])
def test_gemm_job_on_device_resident_tensors(ph, oracle, dev, tmp_path, nodes, policy):
    """The same job with its tensors kept in HBM (`device://<gpu>/0x<address>` storage): LOAD gathers region rows
    by a 2-D device copy, STORE scatters them back, FETCH is an event-tracked peer copy; nothing passes through
    the host.  Executors sit on as many GPUs as the box has (all on GPU 0 otherwise)."""
    import torch
    M, N, K = 1024, 768, 512
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    A, B, C = (torch.from_numpy(x).to(dev) for x in (a, b, c))
    (tmp_path / "gemm.ph").write_text(GEMM_PH)
    (tmp_path / "job.txt").write_text(f"""
source = {tmp_path}/gemm.ph
dim M = {M}
dim N = {N}
dim K = {K}
tensor A = read f32 {M}x{K} {ph.device_uri(A)}
tensor B = read f32 {K}x{N} {ph.device_uri(B)}
tensor C = rmw  f32 {M}x{N} {ph.device_uri(C)}
scalar alpha = f32 0.125
scalar beta = f32 1.5
""")
    job = ph.parse_job(str(tmp_path / "job.txt"))
    prog = ph.Program(job.source)
    prog.check_job(job)
    scalars = {s.name: ph.PhScalar(0, s.dtype, s.bits) for s in job.scalars}
    pl = ph.plan(prog, job.dims, nodes=nodes, scalars=scalars,
                 policy=ph.HOME_LOAD_PEER_FETCH if policy == "fetch" else ph.DIRECT_LOAD)
    pl.validate()
    ndev = torch.cuda.device_count()
    exs = [ph.Executor(n if n < ndev else 0, n, 16 << 20) for n in range(nodes)]
    try:
        assert all(ex.last_run_ms < 0 for ex in exs)
        ph.run_plan(pl, prog, _tensors(job), exs)
        for n, ex in enumerate(exs):
            done = ex.completions()
            assert sorted(d[0] for d in done) == sorted(i.iid for i in pl.node_instrs(n))
            assert all(d[1] == 0 for d in done) and ex.arena_used == 0
            assert ex.last_run_ms >= 0.0
        if policy == "fetch":
            assert sum(ex.served_bytes for ex in exs) == pl.fetch_bytes > 0
    finally:
        for ex in exs:
            ex.close()
    torch.cuda.synchronize()
    assert oracle.rel_frobenius(C.cpu().numpy(), oracle.gemm_rows(a, b, c, 0.125, 1.5)) <= 1e-5
    assert torch.equal(A.cpu(), torch.from_numpy(a))        # inputs untouched
    # a region that leaves the tensor is refused, and so is a malformed address
    I, tid = ph.Instr, ph.tile_id
    with ph.Executor(0, 0, 1 << 20) as ex:
        ex.set_tensors([(ph.device_uri(C), ph.F32, (M, N), ph.RMW)])
        ex.issue([I(iid=1, op=ph.OP_ALLOC, tile=tid(0, 0, 0), shape=(16, 16), data_type=ph.F32),
                  I(iid=2, op=ph.OP_LOAD, tile=tid(0, 0, 0), tensor=0, region_offset=(M - 8, 0), region_shape=(16, 16), deps=(1,))])
        with pytest.raises(ph.PhobosError) as e:
            ex.run()
        assert e.value.code == ph.PH_ERR_INVALID
        with pytest.raises(ph.PhobosError):
            ex.set_tensors([("device://0/zz", ph.F32, (M, N), ph.RMW)])


def test_flash_job_planned_and_executed(ph, oracle, dev, tmp_path):
    """A kernel without a cluster loop is one leaf per query supertile; K and V are loaded whole."""
    Nq, Nk, D = 1024, 640, 128
    q, k, v = (oracle.fp16_round(oracle.lcg_fill_normal(s, n * D)).reshape(n, D) for s, n in ((4, Nq), (5, Nk), (6, Nk)))
    for name, x in zip("qkv", (q, k, v)):
        ph.store_region(f"file://{tmp_path}/{name}.tensor", x.shape, (0, 0), x.astype(np.float16))
    ph.store_region(f"file://{tmp_path}/o.tensor", (Nq, D), (0, 0), np.zeros((Nq, D), np.float16))
    job = ph.parse_job_text(f"""
source = flash.ph
tensor Q = read f16 {Nq}x{D} file://{tmp_path}/q.tensor
tensor K = read f16 {Nk}x{D} file://{tmp_path}/k.tensor
tensor V = read f16 {Nk}x{D} file://{tmp_path}/v.tensor
tensor O = write f16 {Nq}x{D} file://{tmp_path}/o.tensor
scalar scale = f32 0.08838834764831845
""", "job.txt", FLASH_PH)
    prog = ph.Program(job.source)
    prog.check_job(job)
    dims = {"Nq": Nq, "Nk": Nk, "D": D}
    pl = ph.plan(prog, dims, scalars={"scale": ph.PhScalar(0, job.scalars[0].dtype, job.scalars[0].bits)})
    pl.validate()
    assert sum(1 for i in pl.node_instrs(0) if i.op == ph.OP_COMPUTE) == Nq // 512
    with ph.Executor(0, 0, 16 << 20) as ex:
        ph.run_plan(pl, prog, _tensors(job), [ex])
        assert all(d[1] == 0 for d in ex.completions()) and ex.arena_used == 0
    got = ph.load_region(f"file://{tmp_path}/o.tensor", (Nq, D), (0, 0), (Nq, D), dtype=ph.F16).astype(np.float32)
    want = oracle.flash_rows(q, k, v, 0.08838834764831845)
    assert oracle.rel_frobenius(got, want) <= 2e-3


def test_segments_from_the_wire_run_on_the_executor(ph, oracle, dev, tmp_path):
    """What a pod does with a phobos.v1.Segment message: decode, issue, run."""
    M, N, K = 512, 512, 512
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    uris = [f"file://{tmp_path}/{n}.tensor" for n in "abc"]
    for uri, x in zip(uris, (a, b, c)):
        ph.store_region(uri, x.shape, (0, 0), x)
    prog = ph.Program(GEMM_PH)
    pl = ph.plan(prog, {"M": M, "N": N, "K": K}, budget=3 * 256 * 256 * 4,
                 scalars={"alpha": ph.scalar_f32(0, -0.5), "beta": ph.scalar_f32(0, 0.25)})
    messages = [ph.encode_segment(sid, instrs) for sid, instrs, _, _ in pl.segments(0)]
    assert len(messages) > 1
    with ph.Executor(0, 0, 8 << 20) as ex:
        ex.set_tensors([(u, ph.F32, sh, md) for u, sh, md in zip(uris, ((M, K), (K, N), (M, N)), (ph.READ, ph.READ, ph.RMW))])
        for k, entry in enumerate(prog.leaves):
            ex.set_kernel(k, entry)
        for m in messages:
            _, instrs = ph.decode_segment(m)
            ex.issue(instrs)
        ex.run()
        assert all(d[1] == 0 for d in ex.completions())
    got = ph.load_region(uris[2], (M, N), (0, 0), (M, N))
    assert oracle.rel_frobenius(got, oracle.gemm_rows(a, b, c, -0.5, 0.25)) <= 1e-5


SAXPY_PH = """
@cluster(CHUNK in [65536, 1048576])
@autotune(CHUNK in [16, 8192])
kernel saxpy(x: tensor<f32>[N], y: tensor<f32>[N], out: tensor<f32>[N], alpha: f32) {
  let base = program_id(0) * CHUNK
  out[base :+ CHUNK] = alpha * x[base :+ CHUNK] + y[base :+ CHUNK]
}
"""


def test_rank1_job_planned_and_executed(ph, oracle, dev, tmp_path):
    """An elementwise kernel over rank-1 tensors: one leaf per supertile, two nodes, bit-exact result."""
    import torch
    n = 4 * 65536
    x, y = oracle.lcg_fill(42, n), oracle.lcg_fill(43, n)
    for name, v in (("x", x), ("y", y), ("out", np.zeros(n, np.float32))):
        ph.store_region(f"file://{tmp_path}/{name}.tensor", (n,), (0,), v)
    job = ph.parse_job_text(f"""
source = saxpy.ph
dim N = {n}
tensor x = read f32 {n} file://{tmp_path}/x.tensor
tensor y = read f32 {n} file://{tmp_path}/y.tensor
tensor out = write f32 {n} file://{tmp_path}/out.tensor
scalar alpha = f32 0.3
""", "job.txt", SAXPY_PH)
    prog = ph.Program(job.source)
    prog.check_job(job)
    pl = ph.plan(prog, job.dims, nodes=2, scalars={"alpha": ph.PhScalar(0, job.scalars[0].dtype, job.scalars[0].bits)})
    pl.validate()
    assert len(pl.stores) == 4
    ndev = torch.cuda.device_count()
    exs = [ph.Executor(k if k < ndev else 0, k, 4 << 20) for k in range(2)]
    try:
        ph.run_plan(pl, prog, [(t.uri, t.dtype, t.shape, t.mode) for t in job.tensors], exs)
    finally:
        for ex in exs:
            ex.close()
    got = ph.load_region(f"file://{tmp_path}/out.tensor", (n,), (0,), (n,))
    assert np.array_equal(got.view(np.uint32), oracle.saxpy(x, y, 0.3).view(np.uint32))


def test_recovery_plan_redoes_a_dead_nodes_outputs(ph, oracle, dev, tmp_path):
    """Node 1 of two never runs (the failure is made on the host: its segments are simply not issued).
    The recovery plan re-runs its C supertiles on node 0 with fresh instruction ids and bumped tile
    versions, next to what node 0 already did (phobos-sched/src/lib.rs:172-234)."""
    M, N, K = 512, 512, 256
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    uris = [f"file://{tmp_path}/{n}.tensor" for n in "abc"]
    for uri, x in zip(uris, (a, b, c)):
        ph.store_region(uri, x.shape, (0, 0), x)
    prog = ph.Program(GEMM_PH)
    dims = {"M": M, "N": N, "K": K}
    scalars = {"alpha": ph.scalar_f32(0, 2.0), "beta": ph.scalar_f32(0, -0.5)}
    base = ph.plan(prog, dims, nodes=2, scalars=scalars)
    tensors = [(u, ph.F32, sh, md) for u, sh, md in zip(uris, ((M, K), (K, N), (M, N)), (ph.READ, ph.READ, ph.RMW))]
    with ph.Executor(0, 0, 8 << 20) as ex:
        ex.set_tensors(tensors)
        for k, entry in enumerate(prog.leaves):
            ex.set_kernel(k, entry)
        ex.issue(base.node_instrs(0))
        ex.run()
        done = {d[0] for d in ex.completions() if d[1] == 0}
        durable = [(t, lin) for iid, node, t, lin in base.stores if node == 0 and iid in done]
        assert len(durable) == 2
        # half of C is still the original: node 1's supertiles were never computed
        half = ph.load_region(uris[2], (M, N), (0, 0), (M, N))
        want = oracle.gemm_rows(a, b, c, 2.0, -0.5).reshape(M, N)
        lost = [(lin // 2, lin % 2) for _, node, _, lin in base.stores if node == 1]
        for i, j in lost:
            assert np.array_equal(half[i * 256:(i + 1) * 256, j * 256:(j + 1) * 256], c[i * 256:(i + 1) * 256, j * 256:(j + 1) * 256])
        rec = ph.plan(prog, dims, nodes=2, scalars=scalars,
                      recover={"dead": [1], "durable": durable, "version": 1, "iid_base": base.max_iid})
        rec.validate()
        assert sorted(lin for _, _, _, lin in rec.stores) == sorted(lin for _, node, _, lin in base.stores if node == 1)
        ex.issue(rec.node_instrs(0))
        ex.run()
        assert all(d[1] == 0 for d in ex.completions()) and ex.arena_used == 0
    got = ph.load_region(uris[2], (M, N), (0, 0), (M, N))
    assert oracle.rel_frobenius(got, want) <= 1e-5
