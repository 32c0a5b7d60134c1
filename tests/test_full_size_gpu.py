"""Parity at the full benchmark sizes, through the C ABI, on a B200.

The oracle (f64 restatement of the reference verifier, phobos-bench/src/main.rs:386-445, 869-920) takes
seconds per few dozen output rows at these sizes, so each case checks (a) complete sampled output rows
against the oracle under the same relative-Frobenius bound as the small full-matrix cases, (b) the
reference's own 64-point sample criterion restricted to those rows, and (c) a size-independent property
over the WHOLE output.  Inputs are the seeded Lcg streams, generated on the device by the bit-exact
generator and copied back, so both sides see the same bits.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rows(n, count, seed):
    rng = np.random.default_rng(seed)
    r = np.unique(np.concatenate([[0, n - 1], rng.integers(0, n, size=count)])).astype(np.uint64)
    return r


def _device_inputs(ph, torch, dev, M, N, K, ab_dtype, c_dtype, scale):
    A = torch.empty((M, K), dtype=ab_dtype, device=dev)
    B = torch.empty((K, N), dtype=ab_dtype, device=dev)
    C = torch.empty((M, N), dtype=c_dtype, device=dev)
    ph.fill_random(A, seed=1, scale=scale)
    ph.fill_random(B, seed=2, scale=scale)
    ph.fill_random(C, seed=3, scale=scale)
    return A, B, C


def _check_rows(oracle, torch, A, B, C0, C, rows, alpha, beta, tol, ref_tol, ref_floor):
    idx = torch.from_numpy(rows.astype(np.int64)).to(A.device)
    a = A.index_select(0, idx).float().cpu().numpy()
    c0 = C0.index_select(0, idx).float().cpu().numpy()
    b = B.float().cpu().numpy()
    want = oracle.gemm_rows(a, b, c0, alpha, beta)
    got = C.index_select(0, idx).float().cpu().numpy()
    assert np.isfinite(got).all()
    assert oracle.rel_frobenius(got, want) <= tol
    # the reference's criterion: |got - want| / max(|want|, floor) below its tolerance (main.rs:398-402, 438)
    assert oracle.max_rel_floor(got, want, ref_floor) < ref_tol


@pytest.mark.parametrize("with_workspace", [True, False])
def test_headline_gemm_fp16tc_fp32acc_4096(ph, oracle, dev, with_workspace):
    """With the caller's workspace the kernel shares its last 108 tiles between CTA pairs in halves along K
    (the configuration the benchmark times); without it every tile is computed whole."""
    import torch
    M = N = K = 4096
    A, B, C = _device_inputs(ph, torch, dev, M, N, K, torch.float16, torch.float32, 1.0)
    C0 = C.clone()
    ws = None
    if with_workspace:
        nbytes = ph.gemm_workspace_bytes(ph.GEMM_FP16TC_FP32ACC, ph.F16, M, N, K)
        assert nbytes > 0, "4096^3 must qualify for the shared tail"
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
    ph.gemm(A, B, C, 1.0, 0.0, ph.GEMM_FP16TC_FP32ACC, workspace=ws)
    assert ph.device_status() == 0
    # rows from all over, plus rows inside the shared tiles (the second raster band: rows 2048 and up)
    rows = np.unique(np.concatenate([_rows(M, 48, 11), np.arange(2048, 4096, 131, dtype=np.uint64)]))
    _check_rows(oracle, torch, A, B, C0, C, rows, 1.0, 0.0, 2e-3, 1e-2, np.sqrt(K) / 3)
    # whole output: linear in alpha (alpha = 2 doubles every element exactly: beta = 0, power of two)
    C2 = C0.clone()
    ph.gemm(A, B, C2, 2.0, 0.0, ph.GEMM_FP16TC_FP32ACC, workspace=ws)
    assert ph.device_status() == 0
    assert torch.equal(C2, 2.0 * C)
    # and a second launch reproduces the first bit for bit
    C3 = C0.clone()
    ph.gemm(A, B, C3, 1.0, 0.0, ph.GEMM_FP16TC_FP32ACC, workspace=ws)
    assert torch.equal(C3, C)


def test_gemm_fp32_4096(ph, oracle, dev):
    """Both forms of the FFMA kernel at the benchmark size: A read in place, and A read from the transposed
    copy in the caller's workspace."""
    import torch
    M = N = K = 4096
    A, B, C = _device_inputs(ph, torch, dev, M, N, K, torch.float32, torch.float32, 1.0)
    ws = torch.empty((ph.gemm_workspace_bytes(ph.GEMM_FP32, ph.F32, M, N, K),), dtype=torch.uint8, device=dev)
    C0 = C.clone()
    ph.gemm(A, B, C, 0.125, 1.5, ph.GEMM_FP32, workspace=ws)
    assert ph.device_status() == 0
    _check_rows(oracle, torch, A, B, C0, C, _rows(M, 62, 12), 0.125, 1.5, 1e-5, 1e-3, 1.0)
    Cp = C0.clone()
    ph.gemm(A, B, Cp, 0.125, 1.5, ph.GEMM_FP32)
    assert ph.device_status() == 0
    assert torch.equal(Cp, C), "the two forms of the kernel differ"
    # whole output: with beta = 0 and alpha a power of two the result scales exactly
    Ca, Cb = C0.clone(), C0.clone()
    ph.gemm(A, B, Ca, 1.0, 0.0, ph.GEMM_FP32, workspace=ws)
    ph.gemm(A, B, Cb, 0.25, 0.0, ph.GEMM_FP32)
    assert ph.device_status() == 0
    assert torch.equal(Cb, 0.25 * Ca)


def test_gemm_fp16_8192(ph, oracle, dev):
    import torch
    M = N = K = 8192
    A, B, C = _device_inputs(ph, torch, dev, M, N, K, torch.float16, torch.float16, 0.5)
    C0 = C.clone()
    ph.gemm(A, B, C, 1.0, 1.0, ph.GEMM_FP16)
    assert ph.device_status() == 0
    _check_rows(oracle, torch, A, B, C0, C, _rows(M, 30, 13), 1.0, 1.0, 1e-2, 1.5e-1, np.sqrt(K) / 3)
    # whole output: a second launch from the same C_old reproduces it bit for bit
    C2 = C0.clone()
    ph.gemm(A, B, C2, 1.0, 1.0, ph.GEMM_FP16)
    assert ph.device_status() == 0
    assert torch.equal(C2, C)


def test_flash_fp16_b4_h32_s4096_d128(ph, oracle, dev):
    import torch
    BH, S, D = 128, 4096, 128
    scale = 1.0 / np.sqrt(D)
    Q, K, V = (torch.empty((BH, S, D), dtype=torch.float16, device=dev) for _ in range(3))
    for t, seed in ((Q, 4), (K, 5), (V, 6)):
        ph.fill_random(t, seed=seed, normal=True)
    O = torch.full_like(Q, float("nan"))
    ph.flash_attention(Q, K, V, O, scale)
    assert ph.device_status() == 0
    rows = _rows(S, 30, 14)
    ridx = torch.from_numpy(rows.astype(np.int64)).to(dev)
    for h in (0, 37, 127):
        want = oracle.flash_rows(Q[h].float().cpu().numpy(), K[h].float().cpu().numpy(), V[h].float().cpu().numpy(),
                                 scale, rows)
        got = O[h].index_select(0, ridx).float().cpu().numpy()
        assert oracle.rel_frobenius(got, want) <= 2e-3
        assert oracle.max_rel_floor(got, want, 0.1) < 2e-2
    # whole output: every row is a convex combination of the head's V rows, so it lies inside their
    # column-wise range (up to the f16 rounding of P and O) ...
    Of = O.float()
    assert torch.isfinite(Of).all()
    vmin = V.float().amin(dim=1, keepdim=True)
    vmax = V.float().amax(dim=1, keepdim=True)
    assert (Of >= vmin - 2e-2).all() and (Of <= vmax + 2e-2).all()
    # ... and the kernel is linear in V: doubling V (exact in f16) doubles the f32 accumulator exactly, so
    # O doubles bit for bit wherever it is a normal f16 number (a subnormal result rounds on a coarser grid)
    O2 = torch.empty_like(O)
    ph.flash_attention(Q, K, V * 2, O2, scale)
    assert ph.device_status() == 0
    normal = O.abs() >= 2.0 ** -13
    assert torch.equal(O2[normal], (O * 2)[normal])
    assert float((O2.float() - 2 * O.float()).abs().max()) <= 2.0 ** -23


@pytest.mark.parametrize("with_workspace", [False, True])
def test_matmul_cluster_fp32_16384_leaf_chain(ph, oracle, dev, with_workspace):
    """One GPU's view of the partitioned matmul at the full size: the init leaf (C = beta*C) and a chain
    of step leaves (C = alpha*A_k@B_k + C) over K chunks of 2048, as the cluster plan issues them
    (phobos-lang/src/clustergen.rs:1301-1399).  With workspace the step leaf reads a transposed copy of
    its A block (the faster form of the FFMA kernel)."""
    import torch
    M = N = K = 16384
    alpha, beta, kc = 0.125, 1.5, 2048
    A, B, C = _device_inputs(ph, torch, dev, M, N, K, torch.float32, torch.float32, 1.0)
    ws = None
    if with_workspace:
        ws = torch.empty((ph.gemm_workspace_bytes(ph.GEMM_FP32, ph.F32, M, N, kc),), dtype=torch.uint8, device=dev)
    rows = _rows(M, 10, 15)
    idx = torch.from_numpy(rows.astype(np.int64)).to(dev)
    c0 = C.index_select(0, idx).cpu().numpy()
    ph.launch("matmul_init", [C], [ph.scalar_f32(1, beta)], grid=(1, 1, 1), cta=(256, 1, 1))
    for k0 in range(0, K, kc):
        ph.launch("matmul", [A[:, k0:k0 + kc], B[k0:k0 + kc, :], C], [ph.scalar_f32(3, alpha), ph.scalar_f32(4, beta)],
                  grid=(1, 1, 1), cta=(256, 1, 1), kind_hint=ph.KIND_AUTO | ph.LAUNCH_STEP_LEAF, workspace=ws)
    assert ph.device_status() == 0
    a = A.index_select(0, idx).cpu().numpy()
    want = oracle.gemm_rows(a, B.cpu().numpy(), c0, alpha, beta)
    got = C.index_select(0, idx).cpu().numpy()
    assert oracle.rel_frobenius(got, want) <= 1e-5
    assert oracle.max_rel_floor(got, want, 1.0) < 1e-3       # cluster_correctness.rs:124
    assert torch.isfinite(C).all()
