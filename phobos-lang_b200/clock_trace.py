"""SM clock under a leaf workload, at tens of microseconds resolution.

    python phobos-lang_b200/build.py --probes
    python phobos-lang_b200/clock_trace.py [gemm_fp16tc_fp32acc|gemm_fp16|gemm_fp32|flash_fp16] [steps]

A one-thread kernel (csrc/probes/clock_spy.cu) samples (globaltimer, clock64) every 50 us on a side stream
while the leaf runs `steps` times back to back; the ratio of the differences is the SM clock.  nvidia-smi
cannot show this: it samples every few hundred milliseconds, and the clock falls within the first
millisecond of tensor-core load.  Throughput printed here is NOT a benchmark figure: with the sampler
resident a persistent cluster kernel may run one CTA pair short.
"""
from __future__ import annotations

import ctypes
import math
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))


def main() -> None:
    import numpy as np
    import torch
    import __graft_entry__ as entry
    ph = entry.load_package()
    ph.lib()
    spy_path = HERE / "libclock_spy.so"
    if not spy_path.exists():
        raise SystemExit("build the probes first: python phobos-lang_b200/build.py --probes")
    spy = ctypes.CDLL(str(spy_path))
    spy.clock_spy_launch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_void_p]
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm_fp16tc_fp32acc"
    steps = int(sys.argv[2]) if len(sys.argv) > 2 else 20
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)

    if name == "flash_fp16":
        BH, S, D = 128, 4096, 128
        Q, K, V = (torch.empty((BH, S, D), dtype=torch.float16, device=dev) for _ in range(3))
        for t, seed in ((Q, 4), (K, 5), (V, 6)):
            ph.fill_random(t, seed=seed, normal=True)
        O = torch.empty_like(Q)
        flops = 4.0 * BH * S * S * D

        def step(i):
            ph.flash_attention(Q, K, V, O, 1.0 / math.sqrt(D))
    else:
        kind, n, ab, cd, scale, alpha, beta = {
            "gemm_fp16tc_fp32acc": (ph.GEMM_FP16TC_FP32ACC, 4096, torch.float16, torch.float32, 1.0, 1.0, 0.0),
            "gemm_fp16": (ph.GEMM_FP16, 8192, torch.float16, torch.float16, 0.5, 1.0, 1.0),
            "gemm_fp32": (ph.GEMM_FP32, 4096, torch.float32, torch.float32, 1.0, 0.125, 1.5),
        }[name]
        sets = []
        for s in range(3 if n == 4096 else 1):
            A = torch.empty((n, n), dtype=ab, device=dev)
            B = torch.empty((n, n), dtype=ab, device=dev)
            C = torch.empty((n, n), dtype=cd, device=dev)
            for t, seed in ((A, 1), (B, 2), (C, 3)):
                ph.fill_random(t, seed=seed + 3 * s, scale=scale)
            sets.append((A, B, C))
        flops = 2.0 * n * n * n + n * n

        def step(i):
            A, B, C = sets[i % len(sets)]
            ph.gemm(A, B, C, alpha, beta, kind)

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    time.sleep(0.5)                      # idle: the clock returns to its maximum
    n_samples, period_us = 4000, 50      # 200 ms of samples
    buf = torch.zeros(2 * n_samples, dtype=torch.int64, device=dev)
    side = torch.cuda.Stream()
    rc = spy.clock_spy_launch(buf.data_ptr(), n_samples, period_us * 1000, side.cuda_stream)
    if rc != 0:
        raise SystemExit(f"clock_spy_launch failed: {rc}")
    time.sleep(0.002)                    # two idle milliseconds at the head of the trace
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        step(i)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    d = buf.cpu().numpy().reshape(n_samples, 2)
    t = (d[:, 0] - d[0, 0]) / 1e6
    mhz = np.diff(d[:, 1]) / np.diff(d[:, 0]) * 1e3
    print(f"{name}: {steps} steps in {ms:.2f} ms with the sampler resident ({flops * steps / ms / 1e9:.0f} TFLOP/s, "
          "not a benchmark figure)")
    print("SM clock by time since the sampler started (the load starts at ~2 ms):")
    edges = [0, 1, 2, 3, 5, 8, 12, 20, 40, 80, 150, 200]
    for a, b in zip(edges[:-1], edges[1:]):
        m = (t[1:] >= a) & (t[1:] < b)
        if m.any():
            print(f"  {a:4d}-{b:4d} ms: mean {mhz[m].mean():6.0f} MHz, min {mhz[m].min():6.0f}")


if __name__ == "__main__":
    main()
