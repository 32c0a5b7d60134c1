"""`.ph` reader, cluster programs, supertile plans and the supertile autotuner (host only).

The expected numbers restate the reference's own planner tests (phobos-sched/src/lib.rs:1021-1690,
phobos-cluster/src/clustergen.rs:1593-2050, phobos-sched/src/autotune.rs:228-355): a 2x2x2 supertile
matmul is 12 ALLOC / 8 LOAD / 12 COMPUTE / 4 STORE / 12 FREE on one node, and so on.  The kernels below
are written for these tests in the phobos language.
"""
from collections import Counter

import pytest

MATMUL = """
@cluster(SM in [4096, 16384], SN in [4096, 16384], SK in [4096, 16384])
@autotune(SM in [32, 256], SN in [32, 256], SK in [4, 32])
kernel matmul(A: tensor<f32>[M, K], B: tensor<f32>[K, N], C: tensor<f32>[M, N]) {
  let i = program_id(0)
  let j = program_id(1)
  var acc: tile<f32>[SM, SN] = 0.0          // zero start: the init leaf of the chain
  for k0 in range(0, K, SK) {
    acc += dot(A[i * SM :+ SM, k0 :+ SK], B[k0 :+ SK, j * SN :+ SN])
  }
  C[i * SM :+ SM, j * SN :+ SN] = acc
}
"""

GEMM = """
@cluster(SM in [256, 1024], SN in [256, 1024], SK in [256, 1024])
@autotune(SM in [32, 256], SN in [32, 256], SK in [16, 64])
@launch(128)
@tensorcore
kernel gemm(A: tensor<f32>[M, K], B: tensor<f32>[K, N], C: tensor<f32>[M, N], alpha: f32, beta: f32) {
  let i = program_id(0)
  let j = program_id(1)
  var acc: tile<f32>[SM, SN] = 0.0
  for k0 in range(0, K, SK) {
    let a = A[i * SM :+ SM, k0 :+ SK]
    let b = B[k0 :+ SK, j * SN :+ SN]
    acc += dot(a, b)
  }
  let before = C[i * SM :+ SM, j * SN :+ SN]
  C[i * SM :+ SM, j * SN :+ SN] = alpha * acc + beta * before
}
"""

ATTN = """
@cluster(ROWS in [1024, 4096])
@autotune(D in [64], ROWS in [32, 128], COLS in [32, 128])
kernel attn(Q: tensor<f32>[Nq, D], K: tensor<f32>[Nk, D], V: tensor<f32>[Nk, D], O: tensor<f32>[Nq, D], scale: f32) {
  let first = program_id(0) * ROWS
  let q = Q[first :+ ROWS, :]
  var acc: tile<f32>[ROWS, D] = 0.0
  var den: tile<f32>[ROWS, 1] = 0.0
  for c0 in range(0, Nk, COLS) {
    var s: tile<f32>[ROWS, COLS] = dot_t(q, K[c0 :+ COLS, :])
    s = exp(s * scale)
    den += rowsum(s)
    acc += dot(s, V[c0 :+ COLS, :])
  }
  acc = acc / den
  O[first :+ ROWS, :] = acc
}
"""

ADD = """
@cluster(BLOCK in [1048576, 16777216])
@autotune(BLOCK in [16, 4096])
kernel add(a: tensor<f32>[N], b: tensor<f32>[N], c: tensor<f32>[N]) {
  let base = program_id(0) * BLOCK
  c[base :+ BLOCK] = a[base :+ BLOCK] + b[base :+ BLOCK]
}
"""

TILE = 4096 * 4096 * 4


def dims(v):
    return {"M": v, "N": v, "K": v}


def count(ph, pl, node):
    c = Counter(i.op for i in pl.node_instrs(node))
    return {k: c.get(v, 0) for k, v in (("alloc", ph.OP_ALLOC), ("load", ph.OP_LOAD), ("fetch", ph.OP_FETCH),
                                        ("compute", ph.OP_COMPUTE), ("store", ph.OP_STORE), ("free", ph.OP_FREE))}


# ---- declarations --------------------------------------------------------------------------------------
def test_declaration_of_a_kernel(ph):
    p = ph.Program(GEMM)
    assert p.name == "gemm"
    assert [(q.name, q.is_tensor, q.dtype, q.dims) for q in p.params] == [
        ("A", True, ph.F32, ("M", "K")), ("B", True, ph.F32, ("K", "N")), ("C", True, ph.F32, ("M", "N")),
        ("alpha", False, ph.F32, ()), ("beta", False, ph.F32, ())]
    assert p.attrs == ["cluster", "autotune", "launch", "tensorcore"]
    assert p.has_attr("tensorcore") and not p.has_attr("pipeline")
    # two values are bounds searched in doubling steps, longer lists are explicit (ast.rs:58-72)
    assert p.search_choices("cluster", "SM") == [256, 512, 1024]
    assert p.search_choices("autotune", "SK") == [16, 32, 64]
    assert ph.Program(ATTN).search_choices("autotune", "D") == [64]
    assert p.search_choices("cluster", "nope") is None


def test_declaration_errors(ph):
    for bad, what in (("kernel f(A: tensor<f99>[M]) { }", "unknown scalar type"),
                      ("kernel f(A: tensor<f32>[M] { }", "expected ')'"),
                      ("@launch(128 kernel f() { }", "expected ')'"),
                      ("kernel f() { let x = 1 # no such comment\n }", "unexpected character '#'"),
                      ("", "no kernel")):
        with pytest.raises(ph.PhobosError) as e:
            ph.Program(bad)
        assert what in str(e.value), str(e.value)
    with pytest.raises(ph.PhobosError):
        ph.Program(MATMUL, kernel_index=1)


# ---- cluster programs (clustergen) ------------------------------------------------------------------------
def test_matmul_cluster_program(ph):
    """clustergen.rs:1593-1682: grid (M/SM, N/SN), A and B read, C pure output seeded by a zero-init leaf,
    then the k chain with C read-modify-write."""
    p = ph.Program(MATMUL)
    assert p.clustered, p.cluster_error
    assert p.leaves == ["matmul", "matmul_init"]
    assert p.tensor_modes == [ph.READ, ph.READ, ph.WRITE]
    assert p.describe().splitlines() == [
        "program matmul",
        "super SM = 4096 8192 16384", "super SN = 4096 8192 16384", "super SK = 4096 8192 16384",
        "tensor A read dtype1 [M/SM, K/SK]", "tensor B read dtype1 [K/SK, N/SN]", "tensor C write dtype1 [M/SM, N/SN]",
        "leaf matmul cta 256", "leaf matmul_init cta 256",
        "grid 0 M/SM", "grid 1 N/SN",
        "compute leaf 1: C(p0,p1)write scalars",
        "loop k0 over K/SK",
        "  compute leaf 0: A(p0,k0)read B(k0,p1)read C(p0,p1)rmw scalars"]


def test_gemm_cluster_program(ph):
    """clustergen.rs:1737-1796: with `+ beta * c_old` C is read-modify-write, the init leaf carries beta at its
    own position 1 (after C), the step carries the kernel's alpha and beta at 3 and 4; @launch sets the CTA."""
    p = ph.Program(GEMM)
    assert p.clustered, p.cluster_error
    assert p.tensor_modes == [ph.READ, ph.READ, ph.RMW]
    d = p.describe().splitlines()
    assert "leaf gemm cta 128" in d and "leaf gemm_init cta 128" in d
    assert "compute leaf 1: C(p0,p1)rmw scalars beta@1" in d
    assert "  compute leaf 0: A(p0,k0)read B(k0,p1)read C(p0,p1)rmw scalars alpha@3 beta@4" in d


def test_identity_beta_needs_no_init(ph):
    """`... + c_old` keeps C's value: no init leaf, C read-modify-write (clustergen.rs:1192-1200)."""
    p = ph.Program(GEMM.replace("alpha * acc + beta * before", "alpha * acc + before"))
    assert p.clustered, p.cluster_error
    assert p.leaves == ["gemm"] and p.tensor_modes[2] == ph.RMW
    assert not any(line.startswith("compute leaf 1") for line in p.describe().splitlines())


def test_single_leaf_program(ph):
    """clustergen.rs:1925-2005: no cluster loop -> the kernel is one leaf; Q and O are cut along the grid axis,
    K and V are read whole; the scalar keeps its parameter position."""
    p = ph.Program(ATTN)
    assert p.clustered, p.cluster_error
    assert p.leaves == ["attn"]
    assert p.tensor_modes == [ph.READ, ph.READ, ph.READ, ph.WRITE]
    d = p.describe().splitlines()
    assert "tensor Q read dtype1 [Nq/ROWS, D/D]" in d and "tensor K read dtype1 [Nk/Nk, D/D]" in d
    assert "grid 0 Nq/ROWS" in d
    assert d[-1] == "compute leaf 0: Q(p0,:)read K(:,:)read V(:,:)read O(p0,:)write scalars scale@4"


def test_cluster_program_errors(ph):
    """clustergen.rs:2007-2050."""
    cases = (
        (MATMUL.replace("A[i * SM :+ SM", "A[i * SM + 1 :+ SM"), "offset"),
        (MATMUL.replace("@autotune(SM in [32, 256], SN in [32, 256], SK in [4, 32])", "@autotune(SM in [32, 256], SN in [32, 256])"),
         "no @autotune default"),
        (MATMUL.replace("  C[i * SM :+ SM, j * SN :+ SN] = acc\n", "  C[i * SM :+ SM, j * SN :+ SN] = acc\n  C[i * SM :+ SM, j * SN :+ SN] = acc\n"),
         "multiple compute statements"),
        (MATMUL.replace("@cluster(SM in [4096, 16384], SN in [4096, 16384], SK in [4096, 16384])\n", ""), "no @cluster"),
        (MATMUL.replace("B[k0 :+ SK, j * SN :+ SN]", "B[k0 :+ SK, j * SM :+ SM]"), "tiles by both"),
    )
    for src, what in cases:
        p = ph.Program(src)
        assert not p.clustered and what in p.cluster_error, p.cluster_error
        with pytest.raises(ph.PhobosError):
            ph.plan(p, dims(8192))


# ---- plans -----------------------------------------------------------------------------------------------------
def test_matmul_2x2x2_single_node(ph):
    """lib.rs:1021-1096."""
    p = ph.Program(MATMUL)
    pl = ph.plan(p, dims(8192))
    pl.validate()
    assert pl.n_nodes == 1 and len(pl.segments(0)) == 1 and pl.fetch_bytes == 0
    assert count(ph, pl, 0) == {"alloc": 12, "load": 8, "fetch": 0, "compute": 12, "store": 4, "free": 12}
    ins = pl.node_instrs(0)
    assert len(ins) == 48
    c00 = ph.tile_id(2, 0, 0)
    chain = [i for i in ins if i.op == ph.OP_COMPUTE and any(t == c00 for t, _ in i.args)]
    assert [i.kernel for i in chain] == [1, 0, 0]                       # init leaf, then two k steps
    assert chain[0].iid in chain[1].deps and chain[1].iid in chain[2].deps
    assert chain[1].grid == (128, 128, 1) and chain[1].cta == (256, 1, 1)   # 4096 / 32 device tiles, flat CTA
    a01 = ph.tile_id(0, 0, 1)
    free = next(i for i in ins if i.op == ph.OP_FREE and i.tile == a01)
    assert len(free.deps) == 2                                            # after its two consumers
    store = next(i for i in ins if i.op == ph.OP_STORE and i.tile == c00)
    assert store.deps == (chain[2].iid,)
    assert store.region_offset == (0, 0) and store.region_shape == (4096, 4096) and store.tensor == 2
    cfree = next(i for i in ins if i.op == ph.OP_FREE and i.tile == c00)
    assert cfree.deps == (store.iid,)
    assert pl.peak_resident >= 3 * TILE                                   # lib.rs:1441-1449
    assert pl.super_shape(0) == ((4096, 4096), (2, 2))


def test_launch_attribute_sets_the_cta(ph):
    """lib.rs:1098-1111."""
    pl = ph.plan(ph.Program(GEMM), dims(1024), scalars={"alpha": ph.scalar_f32(0, 1.0), "beta": ph.scalar_f32(0, 0.5)})
    assert all(i.cta == (128, 1, 1) for i in pl.node_instrs(0) if i.op == ph.OP_COMPUTE)


def test_two_nodes_home_load_peer_fetch(ph):
    """lib.rs:1113-1185: owner computes by C linear index; A homes to node 0 and crosses once to node 1."""
    p = ph.Program(MATMUL)
    pl = ph.plan(p, dims(8192), nodes=2, policy=ph.HOME_LOAD_PEER_FETCH)
    pl.validate()
    for n in range(2):
        c = count(ph, pl, n)
        assert c["compute"] == 6 and c["store"] == 2
        for i in pl.node_instrs(n):
            if i.op == ph.OP_COMPUTE:
                out = next(t for t, _ in i.args if ph.tile_tensor(t) == 2)
                assert ph.tile_coord(out) % 2 == n
    assert count(ph, pl, 0)["load"] == 6 and count(ph, pl, 1)["load"] == 2
    assert count(ph, pl, 0)["fetch"] == 0 and count(ph, pl, 1)["fetch"] == 4
    assert all(i.from_node == 0 for i in pl.node_instrs(1) if i.op == ph.OP_FETCH)
    serves = [i.expected_serves for i in pl.node_instrs(0) if i.op == ph.OP_FREE and ph.tile_tensor(i.tile) == 0]
    assert serves == [1, 1, 1, 1]
    for n in range(2):
        assert all(i.expected_serves == 0 for i in pl.node_instrs(n) if i.op == ph.OP_FREE and ph.tile_tensor(i.tile) != 0)
    assert pl.fetch_bytes == 4 * TILE                                      # the analytic minimum


def test_two_nodes_direct_load(ph):
    """lib.rs:1187-1221: every node reads what it consumes from storage; 12 LOADs, no peer bytes."""
    pl = ph.plan(ph.Program(MATMUL), dims(8192), nodes=2)
    pl.validate()
    assert pl.fetch_bytes == 0
    for n in range(2):
        c = count(ph, pl, n)
        assert c["fetch"] == 0 and c["load"] == 6
        assert all(i.expected_serves == 0 for i in pl.node_instrs(n) if i.op == ph.OP_FREE)


def test_elementwise_plan(ph):
    """lib.rs:1223-1244."""
    pl = ph.plan(ph.Program(ADD), {"N": 2 * 1048576})
    pl.validate()
    assert count(ph, pl, 0) == {"alloc": 6, "load": 4, "fetch": 0, "compute": 2, "store": 2, "free": 6}


def test_plan_errors(ph):
    p = ph.Program(MATMUL)
    with pytest.raises(ph.PhobosError) as e:                                # lib.rs:1246-1252
        ph.plan(p, dims(10000))
    assert "not a multiple" in str(e.value)
    with pytest.raises(ph.PhobosError) as e:
        ph.plan(p, {"M": 8192, "N": 8192})
    assert "unbound" in str(e.value)
    with pytest.raises(ph.PhobosError) as e:
        ph.plan(p, dims(8192), nodes=0)
    assert "no nodes" in str(e.value)
    with pytest.raises(ph.PhobosError) as e:                                # lib.rs:1352-1367
        ph.plan(ph.Program(ATTN), {"Nq": 4096, "Nk": 2048, "D": 64})
    assert "scalar parameter 'scale' is unbound" in str(e.value)
    with pytest.raises(ph.PhobosError) as e:
        ph.plan(ph.Program(ATTN), {"Nq": 4096, "Nk": 2048, "D": 64}, scalars={"scale": ph.PhScalar(0, ph.I32, 1)})
    assert "bound as type" in str(e.value)


def test_single_leaf_plan(ph):
    """lib.rs:1280-1331."""
    pl = ph.plan(ph.Program(ATTN), {"Nq": 4096, "Nk": 2048, "D": 64}, scalars={"scale": ph.scalar_f32(0, 0.125)})
    pl.validate()
    assert count(ph, pl, 0)["compute"] == 4
    assert pl.super_shape(1) == ((2048, 64), (1, 1)) and pl.super_shape(2)[0] == (2048, 64)
    assert pl.super_shape(0) == ((1024, 64), (4, 1))
    want = ph.scalar_f32(4, 0.125)
    for i in pl.node_instrs(0):
        if i.op == ph.OP_COMPUTE:
            assert [(s.pos, s.dtype, s.bits) for s in i.scalars] == [(want.pos, want.dtype, want.bits)]
            assert i.grid == (1024 // 32, 1, 1)


def test_budget_cuts_segments(ph):
    """lib.rs:1369-1438."""
    p = ph.Program(MATMUL)
    budget = 3 * TILE
    pl = ph.plan(p, dims(8192), budget=budget)
    pl.validate()
    segs = pl.segments(0)
    assert len(segs) > 1
    assert sum(len(s[1]) for s in segs) == 48
    assert all(inc <= budget for _, _, _, inc in segs)
    assert [s[0] for s in segs] == list(range(len(segs)))
    for nodes in (1, 3):                                                    # the saturating case
        pl = ph.plan(p, dims(8192), nodes=nodes, budget=2 * TILE)
        pl.validate()
        assert all(inc <= 2 * TILE for n in range(nodes) for _, _, _, inc in pl.segments(n))
    with pytest.raises(ph.PhobosError) as e:
        ph.plan(p, dims(8192), budget=1024)
    assert "exceeds the memory budget" in str(e.value)


def test_stores_owners_and_recovery(ph):
    """lib.rs:1459-1690: lineage recovery re-runs the chains a dead node owned on the survivors."""
    p = ph.Program(MATMUL)
    base = ph.plan(p, dims(8192), nodes=2)
    assert len(base.stores) == 4
    for _, node, t, lin in base.stores:
        assert t == 2 and node == lin % 2 == base.owner(t, lin)
    rec = ph.plan(p, dims(8192), nodes=2, recover={"dead": [1], "version": 1, "iid_base": base.max_iid})
    rec.validate()
    assert sorted((t, lin) for _, _, t, lin in rec.stores) == [(2, 1), (2, 3)]
    c = count(ph, rec, 0)
    assert c["compute"] == 6 and c["store"] == 2 and c["fetch"] == 0 and c["load"] > 0 and rec.fetch_bytes == 0
    assert rec.node_instrs(1) == []
    # fresh instruction ids and a bumped tile version
    assert min(i.iid for i in rec.node_instrs(0)) == base.max_iid + 1
    assert all(ph.tile_version(i.tile) == 1 for i in rec.node_instrs(0) if i.op == ph.OP_ALLOC)
    # already stored outputs are not redone
    rec = ph.plan(p, dims(8192), nodes=2, recover={"dead": [1], "durable": [(2, 1)], "version": 1, "iid_base": base.max_iid})
    assert sorted((t, lin) for _, _, t, lin in rec.stores) == [(2, 3)]
    # several survivors share the lost chains; a second failure re-recovers what the first recovery placed there
    base4 = ph.plan(p, dims(16384), nodes=4)
    rec = ph.plan(p, dims(16384), nodes=4, recover={"dead": [3], "version": 1, "iid_base": base4.max_iid})
    lost = sorted(lin for _, node, _, lin in base4.stores if node == 3)
    assert sorted(lin for _, _, _, lin in rec.stores) == lost
    assert {node for _, node, _, _ in rec.stores} <= {0, 1, 2} and len({node for _, node, _, _ in rec.stores}) > 1
    with pytest.raises(ph.PhobosError) as e:
        ph.plan(p, dims(8192), nodes=2, recover={"dead": [0, 1]})
    assert "every node has failed" in str(e.value)


# ---- job files against the kernel signature -------------------------------------------------------------------
JOB = """
source = gemm.ph
dim M = 1024
dim N = 512
dim K = 256
tensor A = read f32 1024x256 file:///tmp/a.tensor
tensor B = read f32 256x512 file:///tmp/b.tensor
tensor C = rmw f32 1024x512 file:///tmp/c.tensor
scalar alpha = f32 0.5
scalar beta = f32 1.5
"""


def test_job_bindings_are_checked(ph):
    p = ph.Program(GEMM)
    job = ph.parse_job_text(JOB, "job.txt", GEMM)
    assert job.source == GEMM
    p.check_job(job)
    for bad, what in ((JOB.replace("tensor B = read f32 256x512", "tensor B = read f32 128x512"), "axis 0 is 128 but dim K = 256"),
                      (JOB.replace("tensor C = rmw", "tensor C = read"), "bound read-only"),
                      (JOB.replace("tensor A = read f32", "tensor A = read f16"), "element type"),
                      (JOB.replace("scalar beta = f32 1.5\n", ""), "scalar parameter 'beta' is unbound"),
                      (JOB.replace("scalar alpha = f32 0.5", "scalar alpha = i32 1"), "bound as type"),
                      (JOB.replace("tensor B = read f32 256x512 file:///tmp/b.tensor\n", ""), "'B' is not bound")):
        with pytest.raises(ph.PhobosError) as e:
            p.check_job(ph.parse_job_text(bad, "job.txt", GEMM))
        assert what in str(e.value), str(e.value)


# ---- supertile autotuner ----------------------------------------------------------------------------------------
def test_autotune_ranks_and_prunes(ph):
    """autotune.rs:241-300."""
    p = ph.Program(MATMUL)
    ranked = ph.autotune(p, dims(16384), nodes=2, vram_bytes=16 << 30, link_bytes_per_sec=10e9, leaf_flops_per_sec=10e12)
    assert ranked and len(ranked) <= 27
    assert all(a["makespan_sec"] <= b["makespan_sec"] for a, b in zip(ranked, ranked[1:]))
    assert all(r["peak_resident"] <= 16 << 30 for r in ranked)
    assert set(ranked[0]["supers"]) == {"SM", "SN", "SK"}
    # a grid with fewer output supertiles than nodes leaves a node idle: dropped
    ranked = ph.autotune(p, dims(16384), nodes=4, vram_bytes=64 << 30, link_bytes_per_sec=10e9, leaf_flops_per_sec=10e12)
    for r in ranked:
        assert (16384 // r["supers"]["SM"]) * (16384 // r["supers"]["SN"]) >= 4
    with pytest.raises(ph.PhobosError) as e:
        ph.autotune(p, dims(16384), nodes=2, vram_bytes=1024, link_bytes_per_sec=10e9, leaf_flops_per_sec=10e12)
    assert "no feasible cluster config" in str(e.value)
    # busiest node: every COMPUTE counts 2 x the product of its supertile axes (the init leaves too), at the leaf rate
    best = ph.autotune(p, dims(16384), nodes=2, vram_bytes=180 << 30, link_bytes_per_sec=770e9, leaf_flops_per_sec=50e12)[0]
    want = (2 * 16384 ** 3 + 2 * 16384 ** 2) / 2 / 50e12
    assert abs(best["compute_sec"] - want) / want < 1e-9
    tuned = ph.autotune(ph.Program(ATTN), {"Nq": 8192, "Nk": 2048, "D": 64}, nodes=2, vram_bytes=16 << 30,
                        link_bytes_per_sec=10e9, leaf_flops_per_sec=10e12)
    assert "ROWS" in tuned[0]["supers"]                                     # autotune.rs:321-354
