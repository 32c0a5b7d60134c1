"""Parity of the GEMM leaves with the CPU oracle, through the C ABI, on a B200.

Tolerances are the relative Frobenius bounds of the benchmark contract:
1e-5 (fp32), 2e-3 (f16 operands, f32 accumulate), 1e-2 (pure f16).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_FP32, TOL_F16TC, TOL_F16 = 1e-5, 2e-3, 1e-2


def _inputs(oracle, M, N, K, scale=1.0, seeds=(1, 2, 3)):
    a = oracle.lcg_fill(seeds[0], M * K, scale).reshape(M, K)
    b = oracle.lcg_fill(seeds[1], K * N, scale).reshape(K, N)
    c = oracle.lcg_fill(seeds[2], M * N, scale).reshape(M, N)
    return a, b, c


def _to(dev, x, half=False):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    return t.half() if half else t


# ---------------------------------------------------------------- gemm_fp32 (FFMA)
def _ws32(ph, dev, M, N, K, use):
    """Workspace for the FFMA kernel's transposed copy of A (its faster form), or None (A read in place)."""
    import torch
    if not use:
        return None
    need = ph.gemm_workspace_bytes(ph.GEMM_FP32, ph.F32, M, N, K)
    assert need >= 4 * M * K
    return torch.empty((need,), dtype=torch.uint8, device=dev)


@pytest.mark.parametrize("use_ws", [False, True])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 320), (96, 100, 64), (4, 4, 4), (130, 260, 36),
                                   (1024, 1024, 1024)])
def test_gemm_fp32_matches_oracle(ph, oracle, dev, M, N, K, use_ws):
    a, b, c = _inputs(oracle, M, N, K)
    want = oracle.gemm_rows(a, b, c, 0.125, 1.5)
    A, B, C = _to(dev, a), _to(dev, b), _to(dev, c)
    ph.gemm(A, B, C, 0.125, 1.5, ph.GEMM_FP32, workspace=_ws32(ph, dev, M, N, K, use_ws))
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(C.cpu().numpy(), want) <= TOL_FP32


@pytest.mark.parametrize("M,N,K", [(130, 260, 36), (1000, 520, 4104), (2048, 1024, 272)])
def test_gemm_fp32_both_forms_are_bit_identical(ph, oracle, dev, M, N, K):
    """With workspace the kernel reads a transposed copy of A; the arithmetic per element is the same chain."""
    import torch
    a, b, c = _inputs(oracle, M, N, K)
    A, B = _to(dev, a), _to(dev, b)
    C0, C1 = _to(dev, c), _to(dev, c)
    ph.gemm(A, B, C0, 0.75, -1.25, ph.GEMM_FP32)
    ph.gemm(A, B, C1, 0.75, -1.25, ph.GEMM_FP32, workspace=_ws32(ph, dev, M, N, K, True))
    assert ph.device_status() == 0
    assert torch.equal(C0, C1)
    # a workspace that is too small is not an error: the in-place form runs
    C2 = _to(dev, c)
    ph.gemm(A, B, C2, 0.75, -1.25, ph.GEMM_FP32, workspace=torch.empty((256,), dtype=torch.uint8, device=dev))
    assert torch.equal(C0, C2)


@pytest.mark.parametrize("use_ws", [False, True])
def test_gemm_fp32_is_a_sequential_fma_chain(ph, oracle, dev, use_ws):
    """k ascending, one fma per step, then mul, mul, add: bit-identical to that chain in f32."""
    import torch
    M, N, K = 64, 64, 96
    a, b, c = _inputs(oracle, M, N, K)
    A, B, C = _to(dev, a), _to(dev, b), _to(dev, c)
    ph.gemm(A, B, C, 0.125, 1.5, ph.GEMM_FP32, workspace=_ws32(ph, dev, M, N, K, use_ws))
    # exact emulation of fma.rn in f64: a*b is exact in f64, one rounding to f32 per step
    acc64 = np.zeros((M, N), dtype=np.float32)
    for k in range(K):
        acc64 = (a[:, k:k + 1].astype(np.float64) * b[k:k + 1, :].astype(np.float64)
                 + acc64.astype(np.float64)).astype(np.float32)
    want = (np.float32(0.125) * acc64) + (np.float32(1.5) * c)
    got = C.cpu().numpy()
    # f64 double rounding can differ from a true fma in rare ties; allow a few ulps on a tiny fraction
    mism = np.count_nonzero(got != want)
    assert mism <= got.size // 1000, f"{mism} of {got.size} elements differ from the fma chain"
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("use_ws", [False, True])
def test_gemm_fp32_exact_integer_case_with_guard(ph, dev, use_ws):
    """The reference's masking example: A=(i%7)-3, B=(i%5)-2, 96x64x100, sentinel past the extent
    (phobos-bench/examples/masking.rs:109-152)."""
    import torch
    M, K, N, GUARD, SENT = 96, 64, 100, 4096, -777.0
    a = ((np.arange(M * K) % 7) - 3).astype(np.float32).reshape(M, K)
    b = ((np.arange(K * N) % 5) - 2).astype(np.float32).reshape(K, N)
    want = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    buf = torch.full((M * N + GUARD,), SENT, device=dev)
    buf[:M * N] = 0.0
    C = buf[:M * N].view(M, N)
    ph.gemm(_to(dev, a), _to(dev, b), C, 1.0, 0.0, ph.GEMM_FP32, workspace=_ws32(ph, dev, M, N, K, use_ws))
    assert ph.device_status() == 0
    out = buf.cpu().numpy()
    assert np.array_equal(out[:M * N].reshape(M, N), want)
    assert np.all(out[M * N:] == SENT), "store past the extent"


@pytest.mark.parametrize("use_ws", [False, True])
def test_gemm_fp32_strided_views(ph, oracle, dev, use_ws):
    """Row pitch larger than the row length (a region of a bigger tensor)."""
    M, N, K = 128, 192, 160
    big_a = oracle.lcg_fill(1, M * (K + 32)).reshape(M, K + 32)
    big_b = oracle.lcg_fill(2, K * (N + 64)).reshape(K, N + 64)
    big_c = oracle.lcg_fill(3, M * (N + 64)).reshape(M, N + 64)
    want = oracle.gemm_rows(big_a[:, :K], big_b[:, :N], big_c[:, :N], 2.0, -1.0)
    A, B, C = _to(dev, big_a), _to(dev, big_b), _to(dev, big_c)
    ph.gemm(A[:, :K], B[:, :N], C[:, :N], 2.0, -1.0, ph.GEMM_FP32, workspace=_ws32(ph, dev, M, N, K, use_ws))
    assert ph.device_status() == 0
    got = C.cpu().numpy()
    assert oracle.rel_frobenius(got[:, :N], want) <= TOL_FP32
    assert np.array_equal(got[:, N:], big_c[:, N:]), "columns outside the view were touched"


# ---------------------------------------------------------------- gemm_fp16tc_fp32acc (tcgen05)
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (256, 512, 256), (96, 104, 64), (8, 8, 8),
                                   (200, 328, 136), (1024, 1024, 1024), (384, 64, 192)])
def test_gemm_fp16tc_matches_oracle(ph, oracle, dev, M, N, K):
    a, b, c = _inputs(oracle, M, N, K)
    a16, b16 = oracle.fp16_round(a), oracle.fp16_round(b)
    want = oracle.gemm_rows(a16, b16, c, 1.0, 0.0)
    A, B, C = _to(dev, a16, True), _to(dev, b16, True), _to(dev, c)
    ph.gemm(A, B, C, 1.0, 0.0, ph.GEMM_FP16TC_FP32ACC)
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(C.cpu().numpy(), want) <= TOL_F16TC


def test_gemm_fp16tc_exact_integer_case(ph, dev):
    """Small integers are exact in f16 and in the f32 accumulator: the result must be exact."""
    import torch
    M, K, N = 256, 192, 320
    a = ((np.arange(M * K) % 7) - 3).astype(np.float32).reshape(M, K)
    b = ((np.arange(K * N) % 5) - 2).astype(np.float32).reshape(K, N)
    c = ((np.arange(M * N) % 3) - 1).astype(np.float32).reshape(M, N)
    want = (a.astype(np.int64) @ b.astype(np.int64) * 2 + 3 * c.astype(np.int64)).astype(np.float32)
    C = _to(dev, c)
    ph.gemm(_to(dev, a, True), _to(dev, b, True), C, 2.0, 3.0, ph.GEMM_FP16TC_FP32ACC)
    assert ph.device_status() == 0
    assert np.array_equal(C.cpu().numpy(), want)


def test_gemm_fp16tc_f32_storage_variant(ph, oracle, dev):
    """The .ph signature: f32 A/B rounded RN-even to f16 on the way in (needs workspace)."""
    import torch
    M, N, K = 256, 256, 192
    a, b, c = _inputs(oracle, M, N, K)
    want = oracle.gemm_rows(a, b, c, 0.5, 2.0, round_inputs_f16=True)
    A, B, C = _to(dev, a), _to(dev, b), _to(dev, c)
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm(A, B, C, 0.5, 2.0, ph.GEMM_FP16TC_FP32ACC)
    assert e.value.code == ph.PH_ERR_WORKSPACE
    ws = torch.empty(ph.gemm_workspace_bytes(ph.GEMM_FP16TC_FP32ACC, ph.F32, M, N, K), dtype=torch.uint8, device=dev)
    ph.gemm(A, B, C, 0.5, 2.0, ph.GEMM_FP16TC_FP32ACC, workspace=ws)
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(C.cpu().numpy(), want) <= TOL_F16TC


def test_gemm_beta_zero_still_reads_c(ph, dev):
    """0 * C_old is computed, so a NaN in C propagates (phobos-lang/src/codegen/matmul.rs:393-402)."""
    import torch
    A = torch.ones(128, 64, device=dev, dtype=torch.float16)
    B = torch.ones(64, 128, device=dev, dtype=torch.float16)
    C = torch.zeros(128, 128, device=dev)
    C[5, 7] = float("nan")
    ph.gemm(A, B, C, 1.0, 0.0, ph.GEMM_FP16TC_FP32ACC)
    out = C.cpu().numpy()
    assert np.isnan(out[5, 7]) and out[0, 0] == 64.0


# ---------------------------------------------------------------- gemm_fp16 (f16 accumulate)
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 512), (104, 96, 72), (1024, 1024, 1024)])
def test_gemm_fp16_matches_oracle(ph, oracle, dev, M, N, K):
    a, b, c = _inputs(oracle, M, N, K, scale=0.5)
    a16, b16, c16 = oracle.fp16_round(a), oracle.fp16_round(b), oracle.fp16_round(c)
    want = oracle.gemm_rows(a16, b16, c16, 1.0, 1.0)
    A, B, C = _to(dev, a16, True), _to(dev, b16, True), _to(dev, c16, True)
    ph.gemm(A, B, C, 1.0, 1.0, ph.GEMM_FP16)
    assert ph.device_status() == 0
    got = C.float().cpu().numpy()
    assert oracle.rel_frobenius(got, want) <= TOL_F16
    # the reference's own criterion: sequential f16 model at its 64 sample points, 1.5e-1 normalised
    # by max(|want|, sqrt(K)/3)  (phobos-bench/src/main.rs:649, 663-677)
    pts = oracle.sample_points(M, N)
    model = oracle.gemm_f16acc_points(a16, b16, c16, 1.0, 1.0, pts)
    g = got[pts[:, 0].astype(int), pts[:, 1].astype(int)]
    floor = np.sqrt(K) / 3.0
    assert np.max(np.abs(g - model) / np.maximum(np.abs(model), floor)) < 1.5e-1


# ---------------------------------------------------------------- leaves of the partitioned matmul
def test_matmul_init_and_step_leaves(ph, oracle, dev):
    """init: C = beta*C; steps: C = alpha*A_k@B_k + C; net alpha*A@B + beta*C (clustergen.rs:94-110)."""
    M, N, K, KC = 256, 256, 512, 128
    a, b, c = _inputs(oracle, M, N, K)
    want = oracle.gemm_rows(a, b, c, 0.125, 1.5)
    A, B, C = _to(dev, a), _to(dev, b), _to(dev, c)
    ph.launch("matmul_init", [C], [ph.scalar_f32(1, 1.5)])
    for k0 in range(0, K, KC):
        ph.launch("matmul", [A[:, k0:k0 + KC], B[k0:k0 + KC, :], C],
                  [ph.scalar_f32(3, 0.125), ph.scalar_f32(4, 1.0)], grid=(8, 8, 1))
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(C.cpu().numpy(), want) <= TOL_FP32
    Z = _to(dev, c)
    ph.launch("matmul_init", [Z], [])
    assert float(Z.abs().max()) == 0.0


def test_rejects_bad_descriptors(ph, dev):
    import torch
    A = torch.zeros(64, 64, device=dev)
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm(A, A[:, :62], A, 1.0, 0.0, ph.GEMM_FP32)      # row length not a multiple of 16 bytes
    assert e.value.code == ph.PH_ERR_INVALID
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm(A, A.t(), A, 1.0, 0.0, ph.GEMM_FP32)          # inner stride != 1
    assert e.value.code == ph.PH_ERR_INVALID
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm(A, torch.zeros(32, 64, device=dev), A, 1.0, 0.0, ph.GEMM_FP32)   # K mismatch
    assert e.value.code == ph.PH_ERR_INVALID
    with pytest.raises(ph.PhobosError) as e:
        ph.launch("conv2d", [A], [])
    assert e.value.code == ph.PH_ERR_UNSUPPORTED


def _workspace(ph, dev, kind, a_dtype, M, N, K):
    import torch
    n = ph.gemm_workspace_bytes(kind, a_dtype, M, N, K)
    return torch.empty((max(n, 256),), dtype=torch.uint8, device=dev), n


@pytest.mark.parametrize("shape", [(4864, 1024, 3072), (4864, 1280, 3200), (2560, 2560, 4168), (4864, 1024, 6400),
                                   (5120, 2304, 3080)])
def test_gemm_fp16tc_stream_k_tail(ph, oracle, dev, shape):
    """With a workspace the pair kernel shares out its last rounds of tiles in pieces along K: tiles computed by two
    CTA pairs (one dumps a partial, the other adds it and runs the epilogue) against tiles computed whole.  Tile
    counts just above one round (76, 95, 100) and above two (180); halves of 24 and 25 k-blocks, quarters
    (K = 6400), an odd number of k-blocks (4168 = 65 k-blocks + 8) and a ragged last k-block (3080)."""
    import torch
    M, N, K = shape
    a, b, c = _inputs(oracle, M, N, K)
    a16, b16 = oracle.fp16_round(a), oracle.fp16_round(b)
    rows = np.unique(np.concatenate([np.arange(0, M, 61, dtype=np.uint64), np.arange(M - 512, M, 3, dtype=np.uint64)]))
    want = oracle.gemm_rows(a16, b16, c, 0.5, 1.5, rows=rows)
    A, B = _to(dev, a16, True), _to(dev, b16, True)
    ws, need = _workspace(ph, dev, ph.GEMM_FP16TC_FP32ACC, ph.F16, M, N, K)
    assert need > 0, "this shape must qualify for the stream-K tail"
    results = []
    for use_ws in (True, False, True):       # the third call reuses the workspace (stale partials and flags)
        C = _to(dev, c)
        ph.gemm(A, B, C, 0.5, 1.5, ph.GEMM_FP16TC_FP32ACC, workspace=ws if use_ws else None)
        assert ph.device_status() == 0
        got = C.cpu().numpy()
        assert oracle.rel_frobenius(got[rows.astype(int)], want) <= TOL_F16TC
        results.append(got)
    assert np.array_equal(results[0], results[2]), "a relaunch over a used workspace must give the same bits"
    # with and without the workspace only the summation order of the shared tiles differs (f32 reassociation)
    assert oracle.rel_frobenius(results[0], results[1].astype(np.float64)) <= 1e-4
    # the f16-accumulate kernel shares the scheduler
    ch = oracle.fp16_round(c)
    want16 = oracle.gemm_rows(a16, b16, ch, 1.0, 1.0, rows=rows)
    ws16, need16 = _workspace(ph, dev, ph.GEMM_FP16, ph.F16, M, N, K)
    assert need16 > 0
    Ch = _to(dev, ch, True)
    ph.gemm(A, B, Ch, 1.0, 1.0, ph.GEMM_FP16, workspace=ws16)
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(Ch.float().cpu().numpy()[rows.astype(int)], want16) <= TOL_F16


def test_gemm_fp16tc_f32_storage_with_stream_k(ph, oracle, dev):
    """f32-stored operands: the workspace holds the rounded copies first and the kernel's partial tiles after them;
    a workspace that only fits the copies still works (tiles computed whole)."""
    import torch
    M, N, K = 4864, 1024, 3072
    a, b, c = _inputs(oracle, M, N, K)
    rows = np.arange(0, M, 37, dtype=np.uint64)
    want = oracle.gemm_rows(oracle.fp16_round(a), oracle.fp16_round(b), c, 1.0, 0.0, rows=rows)
    A, B = _to(dev, a), _to(dev, b)
    full = ph.gemm_workspace_bytes(ph.GEMM_FP16TC_FP32ACC, ph.F32, M, N, K)
    staging = 2 * (M * K + K * N)
    assert full > staging
    for nbytes in (full, staging):
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
        C = _to(dev, c)
        ph.gemm(A, B, C, 1.0, 0.0, ph.GEMM_FP16TC_FP32ACC, workspace=ws)
        assert ph.device_status() == 0
        assert oracle.rel_frobenius(C.cpu().numpy()[rows.astype(int)], want) <= TOL_F16TC


def test_host_pipeline_matches_direct_calls(ph, oracle, dev):
    """Calls on pinned host operands, uploads / kernel / download overlapped across calls: same results."""
    import torch
    M, N, K = 512, 384, 256
    pipe = ph.HostPipeline(torch, dev, [((M, K), torch.float32), ((K, N), torch.float32), ((M, N), torch.float32)],
                           lambda a, b, c, stream: ph.gemm(a, b, c, 0.5, 1.5, ph.GEMM_FP32, stream=stream), result_index=2)
    calls = []
    for s in range(5):                      # more calls than buffer sets
        a, b, c = _inputs(oracle, M, N, K, seeds=(10 * s + 1, 10 * s + 2, 10 * s + 3))
        host = [torch.from_numpy(x).pin_memory() for x in (a, b, c)]
        out = torch.empty((M, N), dtype=torch.float32).pin_memory()
        pipe.submit(host, out)
        calls.append((a, b, c, out))
    pipe.join()
    torch.cuda.synchronize()
    assert ph.device_status() == 0
    for a, b, c, out in calls:
        assert oracle.rel_frobenius(out.numpy(), oracle.gemm_rows(a, b, c, 0.5, 1.5)) <= TOL_FP32


@pytest.mark.parametrize("n", [4, 1 << 10, (1 << 20) + 12, 1 << 25])
def test_saxpy_bit_exact(ph, oracle, dev, n):
    """out = alpha*x + y: bit-identical to the reference's own check (a rounded product, then a rounded sum),
    at the reference bench's size 2^25 and at ragged sizes (tail after the unrolled main loop)."""
    import torch
    x, y = oracle.lcg_fill(42, n), oracle.lcg_fill(43, n)
    X, Y = _to(dev, x), _to(dev, y)
    O = torch.full((n,), float("nan"), dtype=torch.float32, device=dev)
    ph.saxpy(X, Y, O, 2.0)
    want = oracle.saxpy(x, y, 2.0)
    assert np.array_equal(O.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # an alpha whose products need rounding separates mul+add from a fused multiply-add
    ph.launch("saxpy", [X, Y, O], [ph.scalar_f32(3, 0.3)])
    want = oracle.saxpy(x, y, 0.3)
    assert np.array_equal(O.cpu().numpy().view(np.uint32), want.view(np.uint32))
    fused = (np.float64(np.float32(0.3)) * x.astype(np.float64) + y.astype(np.float64)).astype(np.float32)
    if n >= 1 << 10:
        assert not np.array_equal(fused, want)
    with pytest.raises(ph.PhobosError):
        ph.saxpy(X, Y[: n - 4] if n > 4 else Y.reshape(2, 2), O, 1.0)
