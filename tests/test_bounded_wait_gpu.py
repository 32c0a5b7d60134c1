"""The bounded-wait policy of the kernels, exercised without breaking a real pipeline.

Every mbarrier wait in the leaf kernels gives up after a time limit, records a site code in the device's
status word and lets the kernel end normally.  phobos_selftest_bounded_wait runs the same wait routine on
a barrier nobody arrives at with a short limit; nothing traps, faults or spins without end.  The
reference's analogues are host side: its stall detector and fetch deadline
(phobos-pod/src/engine.rs:752-775, 825-828)."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SITE_SELFTEST = 0x31


def test_a_wait_that_runs_out_reports_timeout_and_the_device_stays_usable(ph, oracle, dev):
    import torch
    assert ph.device_status() == 0
    t0 = time.time()
    ph.selftest_bounded_wait(1_000_000)          # 1 ms
    with pytest.raises(ph.PhobosError) as e:
        ph.device_status()
    dt = time.time() - t0
    assert e.value.code == ph.PH_ERR_TIMEOUT
    assert f"site 0x{SITE_SELFTEST:x}" in e.value.message
    assert dt < 1.0, f"a 1 ms limit took {dt:.3f} s to report"
    # the status word was cleared by the read, and the context is intact: a normal GEMM runs and is right
    assert ph.device_status() == 0
    M, N, K = 256, 256, 128
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    A, B, C = (torch.from_numpy(x).to(dev) for x in (a, b, c))
    ph.gemm(A, B, C, 0.125, 1.5, ph.GEMM_FP32)
    assert ph.device_status() == 0
    assert oracle.rel_frobenius(C.cpu().numpy(), oracle.gemm_rows(a, b, c, 0.125, 1.5)) <= 1e-5


def test_the_limit_is_the_callers(ph, dev):
    """A longer limit takes longer to run out: the limit passed in is the one that is used."""
    import torch
    torch.cuda.synchronize()
    times = []
    for limit_ns in (2_000_000, 40_000_000):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        ph.selftest_bounded_wait(limit_ns)
        e.record()
        with pytest.raises(ph.PhobosError):
            ph.device_status()
        times.append(s.elapsed_time(e))
    # the limit starts after a short untimed polling phase, so only lower bounds and the difference are firm
    assert times[0] >= 1.5 and times[1] >= 35.0 and times[1] - times[0] >= 25.0 and times[1] < 500.0, times
    with pytest.raises(ph.PhobosError) as ex:
        ph.selftest_bounded_wait(0)
    assert ex.value.code == ph.PH_ERR_INVALID
    with pytest.raises(ph.PhobosError):
        ph.selftest_bounded_wait(5_000_000_000)   # limits above a second are refused


def test_last_launch_clock_reports_a_plausible_sm_clock(ph, dev):
    import torch
    M = N = K = 2048
    A = torch.empty((M, K), device=dev, dtype=torch.float16)
    B = torch.empty((K, N), device=dev, dtype=torch.float16)
    C = torch.zeros((M, N), device=dev)
    ph.fill_random(A, seed=1)
    ph.fill_random(B, seed=2)
    for _ in range(3):
        ph.gemm(A, B, C, 1.0, 0.0, ph.GEMM_FP16TC_FP32ACC)
    cycles, ns = ph.last_launch_clock()
    assert cycles > 0 and ns > 0
    ghz = cycles / ns
    assert 0.5 < ghz < 2.2, (cycles, ns)
