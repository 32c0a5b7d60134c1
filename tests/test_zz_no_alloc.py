"""The no-allocation GEMM entry point, through the C ABI, on a B200.

Some callers of the leaf executor cannot pass a workspace and may not allocate one: a pod that gave
its whole device budget to the tile arena, a serving loop that must stay out of the CUDA allocator.
phobos_gemm_fp16tc_noalloc keeps the scratch for the f16-rounded operands in a fixed array inside
the library instead.  This file checks that it computes exactly what phobos_gemm computes with a
caller workspace, twice in a row (the scratch keeps the previous call's bytes), and that it refuses
problems that do not fit.  It is collected last so that a failure here cannot hide another test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _problem(ph, dev, M, N, K, seed):
    import torch
    A = torch.empty((M, K), device=dev)
    B = torch.empty((K, N), device=dev)
    C = torch.empty((M, N), device=dev)
    ph.fill_random(A, seed=seed)
    ph.fill_random(B, seed=seed + 1)
    ph.fill_random(C, seed=seed + 2)
    return A, B, C


def test_noalloc_matches_the_workspace_entry_point_twice(ph, dev):
    import torch
    # two different problems back to back: the second call finds the first call's bytes in the scratch
    for call, (M, N, K, alpha, beta, seed) in enumerate([(512, 768, 640, 0.5, 2.0, 11), (256, 1024, 384, 1.0, 0.0, 21)]):
        A, B, C = _problem(ph, dev, M, N, K, seed)
        want = C.clone()
        ws = torch.empty(ph.gemm_workspace_bytes(ph.GEMM_FP16TC_FP32ACC, ph.F32, M, N, K), dtype=torch.uint8, device=dev)
        ph.gemm(A, B, want, alpha, beta, ph.GEMM_FP16TC_FP32ACC, workspace=ws)
        got = C.clone()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        ph.gemm_fp16tc_noalloc(A, B, got, alpha, beta)
        assert ph.device_status() == 0
        free_after, _ = torch.cuda.mem_get_info(dev)
        # the first call on a device is the set-up call (the scratch array's module becomes resident,
        # its address is looked up); from then on a call must not take device memory from the driver
        if call > 0:
            assert free_after >= free_before, "the call took device memory from the driver"
        # same kernels on the same rounded operands: bit-identical, which is well inside the 2e-3
        # relative Frobenius bound the other tests use for this GEMM regime
        assert torch.equal(got, want), f"call {call}: max abs diff {(got - want).abs().max().item()}"


def test_noalloc_against_the_oracle(ph, oracle, dev):
    import torch
    M, N, K = 256, 256, 192
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    want = oracle.gemm_rows(a, b, c, 0.5, 2.0, round_inputs_f16=True)
    A, B, C = (torch.from_numpy(x).to(dev) for x in (a, b, c))
    ph.gemm_fp16tc_noalloc(A, B, C, 0.5, 2.0)
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(C.cpu().numpy(), want) <= 2e-3


def test_noalloc_rejects_what_does_not_fit(ph, dev):
    import torch
    M = N = K = 2048          # 2*(M*K + K*N) = 16 MiB > the 8 MiB scratch
    A, B, C = _problem(ph, dev, M, N, K, 31)
    keep = C.clone()
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm_fp16tc_noalloc(A, B, C, 1.0, 0.0)
    assert e.value.code == ph.PH_ERR_WORKSPACE and "built-in scratch" in e.value.message
    assert torch.equal(C, keep)
    H = torch.zeros((256, 256), device=dev, dtype=torch.float16)
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm_fp16tc_noalloc(H, H, torch.zeros((256, 256), device=dev), 1.0, 0.0)
    assert e.value.code == ph.PH_ERR_INVALID


def test_noalloc_validates_before_it_touches_the_scratch(ph, dev):
    """K = 132 is a legal f32 row length (a multiple of 4) but not a legal f16 one (not a multiple of 8):
    the call must be refused before any staging kernel is queued, leaving C as it was."""
    import torch
    A, B, C = _problem(ph, dev, 256, 256, 132, 41)
    keep = C.clone()
    with pytest.raises(ph.PhobosError) as e:
        ph.gemm_fp16tc_noalloc(A, B, C, 1.0, 0.0)
    assert e.value.code == ph.PH_ERR_INVALID
    torch.cuda.synchronize()
    assert torch.equal(C, keep)


def test_noalloc_uses_the_last_byte_of_the_scratch(ph, oracle, dev):
    """2*(M*K + K*N) equal to the scratch size exactly."""
    import torch
    M, N, K = 2048, 2048, 1024
    assert 2 * (M * K + K * N) == ph.NOALLOC_SCRATCH_BYTES
    A, B, C = _problem(ph, dev, M, N, K, 51)
    c0 = C.cpu().numpy()
    ph.gemm_fp16tc_noalloc(A, B, C, 1.0, 1.0)
    assert ph.device_status() == 0
    rows = np.array([0, 1, 777, M - 1], dtype=np.uint64)
    want = oracle.gemm_rows(A.cpu().numpy(), B.cpu().numpy(), c0, 1.0, 1.0, rows=rows, round_inputs_f16=True)
    assert oracle.rel_frobenius(C.cpu().numpy()[rows.astype(int)], want) <= 2e-3
