#!/usr/bin/env python
"""Benchmark of the phobos leaf kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-suite]

Prints ONE JSON line.  Metric: TFLOP/s under the reference's flop conventions
(GEMM 2MNK + MN, phobos-bench/src/main.rs:591; flash 4*Nq*Nk*D per head, main.rs:1032).

N = 1: the headline workload is gemm_fp16tc_fp32acc at M=N=K=4096 (f16 A/B, f32
accumulate and C, alpha 1, beta 0); the other single-GPU configurations
(gemm_fp32 4096^3, gemm_fp16 8192^3, flash_fp16 B4 H32 S4096 D128,
matmul_cluster_fp32 16384^3 on one GPU) are measured the same way and reported
under "suite".  N > 1 (one rank per GPU under torchrun): `value` is the same
headline workload as N independent replicas, one per GPU, timed between barriers
with the maximum over the ranks (weak scaling; the single-GPU leaves do not shard),
so the values at N = 1, 2, 4, 8 form one series.  The one configuration that IS
partitioned across GPUs, matmul_cluster_fp32 16384^3 (2-D C partition, A/B panels
copied over NVLink), is measured in the same run and reported under "partitioned"
(strong scaling; its single-GPU point is suite.matmul_cluster_fp32 of the N = 1 line).

`--impl reference` times the reference's CPU arithmetic for the same workload (the
oracle port of its f64 verifier math, all host threads) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_F16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

KERNEL_FILES = {"gemm_fp16tc_fp32acc": "gemm_tc2.cu", "gemm_fp16": "gemm_tc2.cu", "gemm_fp32": "gemm_f32.cu",
                "matmul_cluster_fp32": "gemm_f32.cu", "flash_fp16": "flash.cu", "saxpy_fp32": "elementwise.cu"}


def _code_only(text):
    """C++ source without comments and blank space, so that a change of wording does not look like a change of
    the kernel.  String literals are kept as they are."""
    out, i, n = [], 0, len(text)
    while i < n:
        c = text[i]
        if c == '"':
            j = i + 1
            while j < n and text[j] != '"':
                j += 2 if text[j] == "\\" else 1
            out.append(text[i:j + 1])
            i = j + 1
        elif text.startswith("//", i):
            while i < n and text[i] != "\n":
                i += 1
        elif text.startswith("/*", i):
            i = text.index("*/", i) + 2
        else:
            out.append(c)
            i += 1
    return "".join("".join(out).split())


def kernel_sha(name):
    """First 12 hex digits of the SHA-256 of the code (comments and blank space removed) of the kernel source that
    serves a workload."""
    import hashlib
    f = ROOT / "phobos-lang_b200" / "csrc" / KERNEL_FILES[name]
    return hashlib.sha256(_code_only(f.read_text()).encode()).hexdigest()[:12]


def ncu_traffic(name):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the workload's kernel from the ncu
    capture recorded in profiles/ncu_traffic.json, with where it came from.  `current` says whether the kernel
    source is still the one that was captured (same SHA-256); a stale figure is reported as such, not as measured."""
    f = ROOT / "profiles" / "ncu_traffic.json"
    if not f.exists() or name not in KERNEL_FILES:
        return None, None
    e = json.loads(f.read_text()).get(name)
    if not e:
        return None, None
    src = {"profile": e.get("profile"), "kernel_source": KERNEL_FILES[name], "captured_sha": e.get("kernel_sha"),
           "current": e.get("kernel_sha") == kernel_sha(name)}
    if e.get("scaled_from"):
        src["scaled_from"] = e["scaled_from"]
    return e["dram_read_bytes"] + e["dram_write_bytes"], src


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


# ---------------------------------------------------------------------------------------------
# clocks: sample nvidia-smi while the timed regions run
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def reader():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        """windows: list of (t0, t1) wall-clock intervals during which timed kernels ran."""
        sm, smax, reasons, power = [], [], set(), []
        for t, line in self.rows:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            under_load = any(a - 0.05 <= t <= b + 0.15 for a, b in windows)
            try:
                clk, mx, pw = float(parts[0]), float(parts[1]), float(parts[2])
            except ValueError:
                continue
            smax.append(mx)
            if under_load:
                sm.append(clk)
                power.append(pw)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm:  # timed regions shorter than the sampling period: fall back to every sample
            for t, line in self.rows:
                parts = [x.strip() for x in line.split(",")]
                try:
                    sm.append(float(parts[0]))
                except (ValueError, IndexError):
                    pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples_under_load": len(power),
                "power_w_max": max(power) if power else None,
                "sampling": "nvidia-smi every 100 ms; the clock inside a burst of tensor-core kernels is lower than "
                            "these samples show: roofline.sm_mhz_in_launch is the clock a CTA of the timed kernel saw"}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
def gemm_flops(M, N, K):
    return 2.0 * M * N * K + M * N


class Ctx:
    def __init__(self, ph, torch, dev, steps, warmup):
        self.ph, self.torch, self.dev, self.steps, self.warmup = ph, torch, dev, steps, warmup
        self.windows = []
        self.cpu_seconds = 1.0   # length of the CPU-baseline sample of the next workload
        self.barrier = None      # N > 1: every timed region starts and ends at a barrier across the ranks
        self.lean = False        # --kernel-only: the timed launches and nothing else

    def time_steps(self, fn_step, steps=None, warmup=None, barrier=None, finish=None):
        """Runs warm-up steps, then times `steps` steps back to back between one pair of CUDA events
        (no event between the steps: an event record between two launches costs ~5 us and keeps the
        next kernel's prologue from overlapping the previous kernel's tail).  Returns (ms per step of
        that region, the same figure as the average launch duration, the shortest single step of a
        second pass in which every step has its own event pair)."""
        torch = self.torch
        steps = self.steps if steps is None else steps
        warmup = self.warmup if warmup is None else warmup
        barrier = barrier or self.barrier
        for i in range(warmup):
            fn_step(i)
        if finish:
            finish()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        t0.record()
        for i in range(steps):
            fn_step(warmup + i)
        if finish:
            finish()       # work on side streams: the closing event waits for it
        t1.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        self.windows.append((w0, time.time()))
        ms = t0.elapsed_time(t1) / steps
        if finish:
            return ms, ms, ms
        n = min(steps, 10)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for i in range(n):
            evs[i][0].record()
            fn_step(warmup + steps + i)
            evs[i][1].record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        return ms, ms, min(a.elapsed_time(b) for a, b in evs)


def pinned_like(torch, t):
    h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
    h.copy_(t)
    return h


def roofline_common(ctx, name, ach, peak_per_clock_flops):
    """Fields every roofline object carries: the DRAM traffic of the kernel with its provenance, and the SM clock
    a CTA of the last timed launch saw (cycles / timer ns) with the fraction of the per-clock peak at that clock."""
    traffic, src = ncu_traffic(name)
    out = {"traffic": traffic if (src and src["current"]) else None, "traffic_source": src}
    if src and not src["current"]:
        out["traffic_stale"] = traffic
    try:
        cyc, ns = ctx.ph.last_launch_clock()
    except Exception:  # noqa: BLE001 - diagnostic only
        cyc, ns = 0, 0
    if cyc and ns:
        mhz = cyc / ns * 1e3
        out["sm_mhz_in_launch"] = round(mhz, 1)
        out["frac_per_clock"] = ach * 1e12 / (peak_per_clock_flops * mhz * 1e6)
    return out


PARITY_TOL = {"gemm_fp32": 1e-5, "matmul_cluster_fp32": 1e-5, "gemm_fp16tc_fp32acc": 2e-3, "gemm_fp16": 1e-2,
              "flash_fp16": 2e-3, "flash_fp32": 2e-3}


def parity_rows(M):
    """Eight complete output rows spread over the tiles (first and last rows, both CTAs of a pair tile, the tiles
    the stream-K tail shares between two CTA pairs)."""
    import numpy as np
    r = sorted({0, min(129, M - 1), M // 4 + 5, M // 2 - 1, M // 2, 3 * M // 4 + 66, M - 130, M - 1})
    return np.array([x for x in r if 0 <= x < M], dtype=np.int64)


def gemm_parity(ctx, name, kind, M, N, K, alpha, beta, A, B, C, scale, workspace):
    """One untimed launch from a freshly generated C, checked on complete rows against the CPU oracle, whose inputs
    come from its own Lcg (seeds 1/2/3) and not from the device: the reference's autotuner verifies every
    configuration on its first launch the same way (phobos-bench/src/autotune.rs:199-201)."""
    import numpy as np
    import oracle
    ph, torch = ctx.ph, ctx.torch
    ph.fill_random(A, seed=1, scale=scale)
    ph.fill_random(B, seed=2, scale=scale)
    ph.fill_random(C, seed=3, scale=scale)
    ph.gemm(A, B, C, alpha, beta, kind, workspace=workspace)
    ph.device_status()
    rows = parity_rows(M)
    got = C[torch.from_numpy(rows).to(C.device)].float().cpu().numpy()
    oracle.use_all_cores()
    half = kind != ph.GEMM_FP32
    a = np.concatenate([oracle.lcg_fill_block(1, int(r) * K, 1, K, K, scale) for r in rows])
    c = np.concatenate([oracle.lcg_fill_block(3, int(r) * N, 1, N, N, scale) for r in rows])
    b = oracle.lcg_fill(2, K * N, scale).reshape(K, N)
    if half:
        a, b = oracle.fp16_round(a), oracle.fp16_round(b)
    if kind == ph.GEMM_FP16:
        c = oracle.fp16_round(c)
    want = oracle.gemm_rows(a, b, c, alpha, beta)
    err = oracle.rel_frobenius(got, want)
    tol = PARITY_TOL[name]
    return {"rel_frobenius": err, "tol": tol, "rows": int(rows.size), "ok": bool(err <= tol)}


def flash_parity(ctx, BH, S, D, Q, K, V, O, scale, workspace, f32_storage):
    import numpy as np
    import oracle
    ph, torch = ctx.ph, ctx.torch
    ph.flash_attention(Q, K, V, O, scale, workspace=workspace)
    ph.device_status()
    oracle.use_all_cores()
    rows = np.array(sorted({0, 127, 128, 255, S // 2 + 3, S - 1}), dtype=np.uint64)
    worst = 0.0
    for h in sorted({0, BH // 2, BH - 1}):
        q, k, v = (oracle.fp16_round(oracle.lcg_fill_normal(seed, S * D, first=h * S * D)).reshape(S, D) for seed in (4, 5, 6))
        want = oracle.flash_rows(q, k, v, scale, rows=rows)
        got = O[h][torch.from_numpy(rows.astype(np.int64)).to(O.device)].float().cpu().numpy()
        worst = max(worst, oracle.rel_frobenius(got, want))
    tol = PARITY_TOL["flash_fp16"]
    return {"rel_frobenius": worst, "tol": tol, "rows": int(rows.size) * 3, "ok": bool(worst <= tol)}


def cublas_bar(ctx, name, M, N, K):
    """The same-box bar the reference prints beside every GEMM (cublasSgemm_v2 / cublasHgemm,
    phobos-bench/src/cublas.rs:106-186, call site main.rs:559-588): torch.matmul, i.e. cuBLAS, on this GPU, in
    the same process, under the same timing rules.  f32 runs with TF32 off.  Not part of the product path."""
    torch, dev = ctx.torch, ctx.dev
    f32 = name in ("gemm_fp32", "matmul_cluster_fp32")
    dt = torch.float32 if f32 else torch.float16
    saved = (torch.backends.cuda.matmul.allow_tf32, torch.get_float32_matmul_precision())
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    f16acc = None
    if name == "gemm_fp16" and hasattr(torch.backends.cuda.matmul, "allow_fp16_accumulation"):
        f16acc = torch.backends.cuda.matmul.allow_fp16_accumulation
        torch.backends.cuda.matmul.allow_fp16_accumulation = True     # cublasHgemm accumulates in f16
    try:
        set_bytes = (M * K + K * N + M * N) * (4 if f32 else 2)
        nsets = max(1, min(4, math.ceil(300e6 / set_bytes)))
        sets = [(torch.randn((M, K), device=dev, dtype=dt) * 0.5, torch.randn((K, N), device=dev, dtype=dt) * 0.5,
                 torch.empty((M, N), device=dev, dtype=dt)) for _ in range(nsets)]

        def step(i):
            a, b, c = sets[i % nsets]
            torch.matmul(a, b, out=c)

        big = M * N * K > 2e12
        ms, _, ms_min = ctx.time_steps(step, steps=3 if big else None, warmup=3)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = saved[0]
        torch.set_float32_matmul_precision(saved[1])
        if f16acc is not None:
            torch.backends.cuda.matmul.allow_fp16_accumulation = f16acc
    del sets
    torch.cuda.empty_cache()
    fl = gemm_flops(M, N, K)
    return {"impl": "cuBLAS via torch.matmul" + (" (f16 accumulation)" if f16acc is not None else "") + (", TF32 off" if f32 else ""),
            "tflops": fl / (ms * 1e-3) / 1e12, "ms_per_step": ms, "ms_min": ms_min}


def bench_gemm(ctx: Ctx, name: str, M: int, N: int, K: int, alpha: float, beta: float, peaks, cpu_baseline=True,
               e2e=True, bar=True):
    ph, torch, dev = ctx.ph, ctx.torch, ctx.dev
    kind = {"gemm_fp32": ph.GEMM_FP32, "matmul_cluster_fp32": ph.GEMM_FP32,
            "gemm_fp16tc_fp32acc": ph.GEMM_FP16TC_FP32ACC, "gemm_fp16": ph.GEMM_FP16}[name]
    ab_dt = torch.float32 if kind == ph.GEMM_FP32 else torch.float16
    c_dt = torch.float16 if kind == ph.GEMM_FP16 else torch.float32
    scale = 0.5 if kind == ph.GEMM_FP16 else 1.0
    set_bytes = (M * K + K * N) * (2 if ab_dt == torch.float16 else 4) + M * N * (2 if c_dt == torch.float16 else 4)
    nsets = max(1, min(4, math.ceil(300e6 / set_bytes)))  # rotate input sets so the working set exceeds L2 (126 MB)
    sets = []
    for s in range(nsets):
        A = torch.empty((M, K), dtype=ab_dt, device=dev)
        B = torch.empty((K, N), dtype=ab_dt, device=dev)
        C = torch.empty((M, N), dtype=c_dt, device=dev)
        ph.fill_random(A, seed=1 + 10 * s, scale=scale)
        ph.fill_random(B, seed=2 + 10 * s, scale=scale)
        ph.fill_random(C, seed=3 + 10 * s, scale=scale)
        sets.append((A, B, C))
    # beta != 0 with |beta| > 1 would grow C over repeated steps: keep a pristine copy and restore outside timing
    pristine = [s[2].clone() for s in sets] if beta != 0.0 else None
    # the pair kernel's scratch for the stream-K tail (partial tiles); the caller owns it, as any workspace
    ws_bytes = ph.gemm_workspace_bytes(kind, ph.F16 if ab_dt == torch.float16 else ph.F32, M, N, K)
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev) if ws_bytes else None

    def step(i):
        A, B, C = sets[i % nsets]
        ph.gemm(A, B, C, alpha, beta, kind, workspace=ws)

    ms_total, ms_launch, ms_min = ctx.time_steps(step)
    ph.device_status()
    if pristine is not None:
        for s, p0 in zip(sets, pristine):
            s[2].copy_(p0)
    flops = gemm_flops(M, N, K)
    out = {"workload": name, "M": M, "N": N, "K": K, "alpha": alpha, "beta": beta,
           "tflops": flops / (ms_total * 1e-3) / 1e12, "ms_per_step": ms_total, "ms_per_launch": ms_launch,
           "ms_min": ms_min, "input_sets": nsets, "workspace_bytes": ws_bytes,
           # with workspace the FFMA GEMM is two launches: A transposed into the workspace, then the kernel
           "launches_per_step": 2 if (kind == ph.GEMM_FP32 and ws_bytes) else 1}
    info = ph.device_info(dev.index or 0)
    ach = flops / (ms_launch * 1e-3) / 1e12
    if kind == ph.GEMM_FP32:
        peak = info.fp32_peak_flops / 1e12
        out["roofline"] = {"bound": "fp32_ffma", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                           "peak_source": f"{info.sm_count} SMs x 128 lanes x 2 x {info.sm_clock_khz / 1e3:.0f} MHz",
                           **roofline_common(ctx, name, ach, info.sm_count * 256.0)}
    else:
        peak = peaks["bf16_tflops"]
        out["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                           "peak_source": f"of {peaks['_source']} (burst cuBLAS bf16)",
                           "frac_of_nominal_2250": ach / NOMINAL_F16_TFLOPS,
                           **roofline_common(ctx, name, ach, info.sm_count * 8192.0)}
    if ctx.lean:
        return out
    out["parity"] = gemm_parity(ctx, name, kind, M, N, K, alpha, beta, *sets[0], scale, ws)
    if bar:
        out["same_box_bar"] = cublas_bar(ctx, name, M, N, K)
    if e2e:
        A, B, C = sets[0]
        hA, hB, hC = pinned_like(torch, A), pinned_like(torch, B), pinned_like(torch, C)
        hOut = torch.empty(C.shape, dtype=C.dtype, device="cpu", pin_memory=True)

        # every step uploads A, B and C_old from pinned host memory and downloads C; the copies of
        # neighbouring steps overlap the kernel (HostPipeline: three streams, two device buffer sets)
        pipe = ph.HostPipeline(torch, dev, [(t.shape, t.dtype) for t in (A, B, C)],
                               lambda a, b, c, stream: ph.gemm(a, b, c, alpha, beta, kind, workspace=ws, stream=stream),
                               result_index=2)

        def e2e_step(i):
            pipe.submit((hA, hB, hC), hOut)

        ms_e2e, _, _ = ctx.time_steps(e2e_step, steps=max(6, min(ctx.steps, 20)), warmup=3, finish=pipe.join)
        del pipe
        out["e2e"] = {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                      "h2d_bytes_per_step": hA.numel() * hA.element_size() + hB.numel() * hB.element_size()
                      + hC.numel() * hC.element_size(),
                      "d2h_bytes_per_step": hOut.numel() * hOut.element_size()}
    if cpu_baseline:
        out["cpu_baseline"] = cpu_gemm_baseline(name, M, N, K, alpha, beta, min_seconds=ctx.cpu_seconds)
    del sets
    torch.cuda.empty_cache()
    return out


def bench_flash(ctx: Ctx, BH: int, S: int, D: int, peaks, cpu_baseline=True, e2e=True, f32_storage=False):
    """flash_fp16, or with f32_storage flash_fp32: f32 Q/K/V/O, staged to f16 by a convert pass inside the
    timed step, the same tensor-core kernel, O written as f32 by its epilogue."""
    ph, torch, dev = ctx.ph, ctx.torch, ctx.dev
    scale = 1.0 / math.sqrt(D)
    dt = torch.float32 if f32_storage else torch.float16
    Q, K, V = (torch.empty((BH, S, D), dtype=dt, device=dev) for _ in range(3))
    for t, seed in ((Q, 4), (K, 5), (V, 6)):
        ph.fill_random(t, seed=seed, normal=True)   # N(0,1): Box-Muller over the Lcg stream (no reference analogue)
    O = torch.empty_like(Q)
    ws = None
    if f32_storage:
        ws = torch.empty((ph.flash_workspace_bytes(ph.F32, BH, S, S, D),), dtype=torch.uint8, device=dev)

    def step(i):
        ph.flash_attention(Q, K, V, O, scale, workspace=ws)

    ms_total, ms_launch, ms_min = ctx.time_steps(step)
    ph.device_status()
    flops = 4.0 * BH * S * S * D
    ach = flops / (ms_launch * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    out = {"workload": "flash_fp32" if f32_storage else "flash_fp16", "launches_per_step": 4 if f32_storage else 1, "batch_heads": BH, "seq_len": S, "head_dim": D,
           "tflops": flops / (ms_total * 1e-3) / 1e12, "ms_per_step": ms_total, "ms_per_launch": ms_launch,
           "ms_min": ms_min, "exp_per_s": BH * S * S / (ms_launch * 1e-3),
           "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                        "peak_source": f"of {peaks['_source']} (burst cuBLAS bf16)",
                        "frac_of_nominal_2250": ach / NOMINAL_F16_TFLOPS,
                        **roofline_common(ctx, "flash_fp32" if f32_storage else "flash_fp16", ach,
                                          ph.device_info(dev.index or 0).sm_count * 8192.0)}}
    if ctx.lean:
        return out
    out["parity"] = flash_parity(ctx, BH, S, D, Q, K, V, O, scale, ws, f32_storage)
    if f32_storage:
        out["launches_per_step"] = 4      # three f32 -> f16 staging passes and the attention kernel
    if e2e:
        hQ, hK, hV = (pinned_like(torch, t) for t in (Q, K, V))
        hO = torch.empty(O.shape, dtype=O.dtype, device="cpu", pin_memory=True)

        pipe = ph.HostPipeline(torch, dev, [(t.shape, t.dtype) for t in (Q, K, V, O)],
                               lambda q, k, v, o, stream: ph.flash_attention(q, k, v, o, scale, workspace=ws, stream=stream),
                               result_index=3)

        def e2e_step(i):
            pipe.submit((hQ, hK, hV, None), hO)

        ms_e2e, _, _ = ctx.time_steps(e2e_step, steps=max(6, min(ctx.steps, 20)), warmup=3, finish=pipe.join)
        del pipe
        nb = Q.numel() * Q.element_size()
        out["e2e"] = {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                      "h2d_bytes_per_step": 3 * nb, "d2h_bytes_per_step": nb}
    if cpu_baseline:
        out["cpu_baseline"] = cpu_flash_baseline(BH, S, D, min_seconds=ctx.cpu_seconds)
    return out


def bench_saxpy(ctx: Ctx, n: int, peaks, cpu_baseline=True, e2e=True):
    """saxpy_fp32 at the reference bench's size (n = 2^25, alpha = 2, phobos-bench/src/main.rs:1198-1199):
    12 bytes of HBM traffic per element, 2 flop."""
    ph, torch, dev = ctx.ph, ctx.torch, ctx.dev
    alpha = 2.0
    sets = []
    for s in range(2):     # two input sets: 768 MB in rotation, every launch reads from HBM
        x, y = (torch.empty((n,), dtype=torch.float32, device=dev) for _ in range(2))
        ph.fill_random(x, seed=42 + 2 * s)
        ph.fill_random(y, seed=43 + 2 * s)
        sets.append((x, y, torch.empty((n,), dtype=torch.float32, device=dev)))

    def step(i):
        x, y, o = sets[i % len(sets)]
        ph.saxpy(x, y, o, alpha)

    ms_total, ms_launch, ms_min = ctx.time_steps(step)
    ph.device_status()
    flops, nbytes = 2.0 * n, 12.0 * n
    ach = nbytes / (ms_launch * 1e-3) / 1e9
    out = {"workload": "saxpy_fp32", "n": n, "alpha": alpha, "tflops": flops / (ms_total * 1e-3) / 1e12,
           "gbytes_per_s": nbytes / (ms_total * 1e-3) / 1e9, "ms_per_step": ms_total, "ms_per_launch": ms_launch,
           "ms_min": ms_min, "input_sets": len(sets),
           "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                        "peak_source": f"of {peaks['_source']} (STREAM-style copy)",
                        **{k: v for k, v in roofline_common(ctx, "saxpy_fp32", 0.0, 1.0).items() if k.startswith("traffic")}}}
    if ctx.lean:
        return out
    if e2e:
        x, y, o = sets[0]
        hx, hy = pinned_like(torch, x), pinned_like(torch, y)
        ho = torch.empty(o.shape, dtype=o.dtype, device="cpu", pin_memory=True)
        pipe = ph.HostPipeline(torch, dev, [(t.shape, t.dtype) for t in (x, y, o)],
                               lambda a, b, c, stream: ph.saxpy(a, b, c, alpha, stream=stream), result_index=2)

        def e2e_step(i):
            pipe.submit((hx, hy, None), ho)

        ms_e2e, _, _ = ctx.time_steps(e2e_step, steps=max(6, min(ctx.steps, 20)), warmup=3, finish=pipe.join)
        del pipe
        out["e2e"] = {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                      "h2d_bytes_per_step": 8 * n, "d2h_bytes_per_step": 4 * n}
    if cpu_baseline:
        import oracle
        xh, yh = oracle.lcg_fill(42, n), oracle.lcg_fill(43, n)
        reps, t0 = 0, time.time()
        while True:
            oracle.saxpy(xh, yh, alpha)
            reps += 1
            dt = time.time() - t0
            if dt >= ctx.cpu_seconds or reps >= 64:
                break
        out["cpu_baseline"] = {"value": flops * reps / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
                               "sample": f"{reps} x (all {n} elements; f32 multiply then add, OpenMP); {dt:.2f} s"}
    del sets
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle (port of the reference's f64 verifier arithmetic), bounded sample
# ---------------------------------------------------------------------------------------------
def cpu_gemm_baseline(name, M, N, K, alpha, beta, budget_flops=4e11, min_seconds=1.0):
    import numpy as np
    import oracle
    oracle.use_all_cores()
    rows_n = int(max(64, min(M, budget_flops / (2.0 * N * K))))
    rows_n -= rows_n % 4
    rows = np.arange(rows_n, dtype=np.uint64)
    half = name in ("gemm_fp16tc_fp32acc", "gemm_fp16")
    scale = 0.5 if name == "gemm_fp16" else 1.0
    a = oracle.lcg_fill(1, rows_n * K, scale).reshape(rows_n, K)
    b = oracle.lcg_fill(2, K * N, scale).reshape(K, N)
    c = oracle.lcg_fill(3, rows_n * N, scale).reshape(rows_n, N)
    if half:
        a, b = oracle.fp16_round(a), oracle.fp16_round(b)
    reps = 0
    t0 = time.time()
    while True:   # the same rows again until the sample is long enough to time
        oracle.gemm_rows(a, b, c, alpha, beta, rows=rows)
        reps += 1
        dt = time.time() - t0
        if dt >= min_seconds or reps >= 64:
            break
    fl = (2.0 * rows_n * N * K + rows_n * N) * reps
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"{reps} x ({rows_n} of {M} output rows x all {N} columns, K={K}; f64 accumulate, OpenMP); {dt:.2f} s"}


def cpu_flash_baseline(BH, S, D, rows_n=4096, min_seconds=1.0):
    import numpy as np
    import oracle
    oracle.use_all_cores()
    q = oracle.fp16_round(oracle.lcg_fill_normal(4, S * D)).reshape(S, D)
    k = oracle.fp16_round(oracle.lcg_fill_normal(5, S * D)).reshape(S, D)
    v = oracle.fp16_round(oracle.lcg_fill_normal(6, S * D)).reshape(S, D)
    rows_n = min(rows_n, S)
    rows = np.arange(0, S, S // rows_n, dtype=np.uint64)[:rows_n]
    reps = 0
    t0 = time.time()
    while True:
        oracle.flash_rows(q, k, v, 1.0 / math.sqrt(D), rows=rows)
        reps += 1
        dt = time.time() - t0
        if dt >= min_seconds or reps >= 64:
            break
    fl = 4.0 * rows.size * S * D * reps
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"{reps} x ({rows.size} of {BH * S} query rows, one head, all {S} keys; f64 online softmax, OpenMP); {dt:.2f} s"}


# ---------------------------------------------------------------------------------------------
# N > 1: partitioned matmul_cluster_fp32
# ---------------------------------------------------------------------------------------------
def bench_partitioned(ctx: Ctx, world: int, rank: int, MNK: int, alpha: float, beta: float):
    import torch.distributed as dist
    ph, torch, dev = ctx.ph, ctx.torch, ctx.dev
    part = sys.modules[ph.__name__ + ".partition"]
    kc = part.default_k_chunk(MNK, world)
    plan = part.plan_partition(MNK, MNK, MNK, world, k_chunk=kc)
    row_pg, col_pg = part.make_groups(plan, rank)
    row0, mb, col0, nb = plan.c_block(rank)
    ak0, aw = plan.a_shard_k(rank)
    bk0, bh = plan.b_shard_k(rank)
    # home shards, generated in place from the global Lcg streams (A seed 1, B seed 2, C seed 3)
    a_rows = torch.empty((mb, aw), dtype=torch.float32, device=dev)
    b_shard = torch.empty((bh, nb), dtype=torch.float32, device=dev)
    c0 = torch.empty((mb, nb), dtype=torch.float32, device=dev)
    fill_block(ph, a_rows, 1, row0, ak0, MNK)
    fill_block(ph, b_shard, 2, bk0, col0, MNK)
    fill_block(ph, c0, 3, row0, col0, MNK)
    a_shard = a_rows.reshape(mb, aw // kc, kc).permute(1, 0, 2).contiguous()
    del a_rows
    c_block = c0.clone()
    comm, comp = torch.cuda.Stream(), torch.cuda.Stream()
    bufs = part.alloc_buffers(plan, a_shard, b_shard)
    leaf_init, leaf_step = part.cuda_leaves()
    # exchange: peer copies out of the home ranks' shards (no collective, no SMs); PHOBOS_EXCHANGE=nccl
    # selects the broadcast form instead
    peers, exchange = None, "nccl"
    if os.environ.get("PHOBOS_EXCHANGE", "p2p") == "p2p":
        # every rank must take the same path: agree on whether symmetric memory came up everywhere
        try:
            peers = part.PeerShards(plan, rank, a_shard, b_shard)
            ok = torch.ones(1, device=dev)
        except Exception as ex:  # noqa: BLE001 - reported, then the collective form is used
            print(f"rank {rank}: symmetric memory unavailable ({ex}); using NCCL broadcasts", file=sys.stderr)
            peers, ok = None, torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            peers = None
        exchange = "p2p" if peers is not None else "nccl"
    pa, pb = (peers.a, peers.b) if peers is not None else (a_shard, b_shard)

    def step(i):
        part.run_partitioned(plan, rank, pa, pb, c_block, alpha, beta, leaf_init, leaf_step, row_pg, col_pg,
                             comm_stream=comm, compute_stream=comp, buffers=bufs, peers=peers)
        torch.cuda.current_stream().wait_stream(comp)
        torch.cuda.current_stream().wait_stream(comm)

    def reset():
        c_block.copy_(c0)

    def timed_step(i):
        reset()
        step(i)

    # C is restored before every step; the restore (a device copy of the C block) is part of the step,
    # as the reference's per-launch C reset is (phobos-bench/src/main.rs:267-279)
    ms_total, ms_launch, ms_min = ctx.time_steps(timed_step, barrier=dist.barrier)
    ph.device_status()
    t = torch.tensor([ms_total], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops = gemm_flops(MNK, MNK, MNK)

    # upper bound without any exchange (the reference's DirectLoad ingest: every rank holds the whole A row
    # panel and B column panel it consumes): the same init + step leaves over resident panels
    a_full = torch.empty((mb, MNK), dtype=torch.float32, device=dev)
    b_full = torch.empty((MNK, nb), dtype=torch.float32, device=dev)
    fill_block(ph, a_full, 1, row0, 0, MNK)
    fill_block(ph, b_full, 2, 0, col0, MNK)

    def direct_step(i):
        c_block.copy_(c0)
        leaf_init(c_block, beta)
        for k0 in range(0, MNK, kc):
            leaf_step(a_full[:, k0:k0 + kc], b_full[k0:k0 + kc, :], c_block, alpha)

    ms_direct, _, _ = ctx.time_steps(direct_step, steps=max(2, min(ctx.steps, 3)), warmup=1, barrier=dist.barrier)
    t = torch.tensor([ms_direct], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_direct = float(t.item())
    del a_full, b_full
    torch.cuda.empty_cache()

    # e2e: shards come from pinned host memory every step, the C block goes back
    hA, hB, hC = pinned_like(torch, a_shard), pinned_like(torch, b_shard), pinned_like(torch, c0)
    hOut = torch.empty(c0.shape, dtype=c0.dtype, device="cpu", pin_memory=True)

    def e2e_step(i):
        # the uploaded shards are exchanged by broadcast here: a collective orders every rank's upload
        # before its peers read it, which the one-sided copies of the timed path do not need
        a_shard.copy_(hA, non_blocking=True)
        b_shard.copy_(hB, non_blocking=True)
        c_block.copy_(hC, non_blocking=True)
        comp.wait_stream(torch.cuda.current_stream())
        part.run_partitioned(plan, rank, a_shard, b_shard, c_block, alpha, beta, leaf_init, leaf_step, row_pg, col_pg,
                             comm_stream=comm, compute_stream=comp, buffers=bufs)
        torch.cuda.current_stream().wait_stream(comp)
        torch.cuda.current_stream().wait_stream(comm)
        hOut.copy_(c_block, non_blocking=True)

    ms_e2e, _, _ = ctx.time_steps(e2e_step, steps=max(3, min(ctx.steps, 5)), warmup=3, barrier=dist.barrier)
    t = torch.tensor([ms_e2e], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())
    # parity: one clean run from c0, then complete rows of this rank's C block against the CPU oracle on the same
    # Lcg streams (A seed 1, B seed 2, C seed 3), as the reference checks its cluster matmul at this size by
    # recomputing sampled cells in f64 (phobos-pod/examples/cluster_correctness.rs:97-125, 252-273)
    import numpy as np
    import oracle
    c_block.copy_(c0)
    step(0)
    torch.cuda.synchronize()
    ph.device_status()
    lrows = np.array(sorted({0, 1, mb // 3 + 7, mb // 2 - 1, mb // 2, mb - 130, mb - 2, mb - 1}), dtype=np.int64)
    got = c_block[torch.from_numpy(lrows).to(dev)].cpu().numpy()
    oracle.use_all_cores()
    a_rows_h = np.concatenate([oracle.lcg_fill_block(1, (row0 + int(r)) * MNK, 1, MNK, MNK) for r in lrows])
    c_rows_h = np.concatenate([oracle.lcg_fill_block(3, (row0 + int(r)) * MNK + col0, 1, nb, MNK) for r in lrows])
    b_blk_h = oracle.lcg_fill_block(2, col0, MNK, nb, MNK)
    want = oracle.gemm_rows(a_rows_h, b_blk_h, c_rows_h, alpha, beta)
    err = oracle.rel_frobenius(got, want)
    del b_blk_h, want
    t = torch.tensor([err], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    err = float(t.item())
    parity = {"rel_frobenius": err, "tol": 1e-5, "rows": int(lrows.size) * world, "ok": bool(err <= 1e-5)}

    # strong-scaling efficiency T1 / (N * TN): the same problem as one init leaf and the same chain of step leaves
    # over K chunks on one GPU (rank 0), timed in this process while the other ranks wait
    ms_one = None
    if rank == 0:
        a1 = torch.empty((MNK, MNK), dtype=torch.float32, device=dev)
        b1 = torch.empty((MNK, MNK), dtype=torch.float32, device=dev)
        c1 = torch.empty((MNK, MNK), dtype=torch.float32, device=dev)
        fill_block(ph, a1, 1, 0, 0, MNK)
        fill_block(ph, b1, 2, 0, 0, MNK)
        fill_block(ph, c1, 3, 0, 0, MNK)

        def one_step(i):
            leaf_init(c1, beta)
            for k0 in range(0, MNK, kc):
                leaf_step(a1[:, k0:k0 + kc], b1[k0:k0 + kc, :], c1, alpha)

        ms_one, _, _ = ctx.time_steps(one_step, steps=3, warmup=1, barrier=lambda: None)
        del a1, b1, c1
        torch.cuda.empty_cache()
    dist.barrier()
    info = ph.device_info(dev.index or 0)
    peak = info.fp32_peak_flops / 1e12 * world
    ach = flops / (ms * 1e-3) / 1e12
    out = {"workload": "matmul_cluster_fp32", "parity": parity,
           "one_gpu_ms_per_step": ms_one, "efficiency": (ms_one / (world * ms)) if ms_one else None, "M": MNK, "N": MNK, "K": MNK, "alpha": alpha, "beta": beta,
           "grid": f"{plan.pr}x{plan.pc}", "k_chunk": kc, "steps_per_rank": len(plan.steps), "exchange": exchange,
           "tflops": ach, "ms_per_step": ms,
           "peer_bytes_per_step": plan.total_peer_bytes(), "peer_bytes_per_rank": plan.recv_bytes(rank),
           "direct_load_bound": {"tflops": flops / (ms_direct * 1e-3) / 1e12, "ms_per_step": ms_direct,
                                 "note": "panels resident on every rank, no exchange: upper bound for the partitioned run"},
           "roofline": {"bound": "fp32_ffma", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                        "peak_source": f"{world} x {info.sm_count} SMs x 128 lanes x 2 x {info.sm_clock_khz / 1e3:.0f} MHz",
                        "nvlink_floor_ms": plan.recv_bytes(rank) / 770e9 * 1e3, "traffic": None},
           "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": world * (hA.numel() + hB.numel() + hC.numel()) * 4,
                   "d2h_bytes_per_step": world * hOut.numel() * 4},
           # per step and rank: the init leaf, then for every K chunk the transposition of the A block and the FFMA kernel
           "gpu_launches": (1 + 2 * len(plan.steps)) * ctx.steps * world}
    return out


MATMUL_PH = """
@cluster(TM in [4096, 16384], TN in [4096, 16384], TK in [4096, 16384])
@autotune(TM in [32, 128], TN in [32, 128], TK in [4, 16])
kernel matmul(A: tensor<f32>[M, K], B: tensor<f32>[K, N], C: tensor<f32>[M, N], alpha: f32, beta: f32) {
  let bi = program_id(0)
  let bj = program_id(1)
  var acc: tile<f32>[TM, TN] = 0.0
  for kk in range(0, K, TK) {
    acc += dot(A[bi * TM :+ TM, kk :+ TK], B[kk :+ TK, bj * TN :+ TN])
  }
  let old = C[bi * TM :+ TM, bj * TN :+ TN]
  C[bi * TM :+ TM, bj * TN :+ TN] = alpha * acc + beta * old
}
"""


def bench_plan_driven(ctx: Ctx, world: int, MNK: int, alpha: float, beta: float, steps: int = 3, warm: int = 2):
    """The same partitioned matmul through the C ABI only (rank 0 drives it): job text -> phobos_plan_make
    (HomeLoadPeerFetch over `world` nodes, the reference's default supertiles) -> one executor per GPU, tensors
    resident in GPU 0's HBM (device:// storage), LOAD / FETCH / STORE as device and peer copies, leaves by entry
    name.  Time: the longest executor run, on the device (events of each executor's own streams)."""
    import numpy as np
    import oracle
    ph, torch, dev = ctx.ph, ctx.torch, ctx.dev
    # A, B and C each live whole in one GPU's HBM, on different GPUs where there are that many, so that the
    # LOADs of the job do not all leave through one GPU's links
    homes = [torch.device("cuda", k % world) for k in range(3)]
    tensors_dev = []
    for seed, home in zip((1, 2, 3), homes):
        with torch.cuda.device(home):
            t = torch.empty((MNK, MNK), dtype=torch.float32, device=home)
            if seed != 3:
                fill_block(ph, t, seed, 0, 0, MNK)
            tensors_dev.append(t)
    A, B, C = tensors_dev
    job = ph.parse_job_text(f"""
source = matmul.ph
dim M = {MNK}
dim N = {MNK}
dim K = {MNK}
tensor A = read f32 {MNK}x{MNK} {ph.device_uri(A)}
tensor B = read f32 {MNK}x{MNK} {ph.device_uri(B)}
tensor C = rmw  f32 {MNK}x{MNK} {ph.device_uri(C)}
scalar alpha = f32 {alpha}
scalar beta = f32 {beta}
""", "bench job", MATMUL_PH)
    prog = ph.Program(MATMUL_PH)
    prog.check_job(job)
    scalars = {sc.name: ph.PhScalar(0, sc.dtype, sc.bits) for sc in job.scalars}
    # supertiles: the planner's own cost model (phobos_autotune: NVLink rate, the measured rate of the FFMA leaf, the
    # arena as the memory limit) ranks the @cluster choices; the best one is planned
    arena = 12 << 30
    ranked = ph.autotune(prog, job.dims, world, arena, 770e9, 64e12)
    supers = ranked[0]["supers"] if ranked else None
    pl = ph.plan(prog, job.dims, supers=supers, nodes=world, scalars=scalars, policy=ph.HOME_LOAD_PEER_FETCH)
    pl.validate()
    tensors = [(t.uri, t.dtype, t.shape, t.mode) for t in job.tensors]
    # the executors live as long as a pod's would: the untimed runs also grow each one's workspace
    times, served = [], 0
    exs = [ph.Executor(n, n, arena) for n in range(world)]
    try:
        for it in range(warm + steps):
            with torch.cuda.device(homes[2]):
                fill_block(ph, C, 3, 0, 0, MNK)
            for home in homes:
                torch.cuda.synchronize(home)
            before = sum(ex.served_bytes for ex in exs)
            ph.run_plan(pl, prog, tensors, exs)
            if it >= warm:
                per_node = [round(ex.last_run_ms, 3) for ex in exs]
                times.append(max(per_node))
            served = sum(ex.served_bytes for ex in exs) - before
    finally:
        for ex in exs:
            ex.close()
    for n in range(world):
        torch.cuda.synchronize(n)
        with torch.cuda.device(n):
            ph.device_status()
    rows = parity_rows(MNK)
    got = C[torch.from_numpy(rows).to(C.device)].cpu().numpy()
    oracle.use_all_cores()
    a = np.concatenate([oracle.lcg_fill_block(1, int(r) * MNK, 1, MNK, MNK) for r in rows])
    c = np.concatenate([oracle.lcg_fill_block(3, int(r) * MNK, 1, MNK, MNK) for r in rows])
    b = oracle.lcg_fill(2, MNK * MNK).reshape(MNK, MNK)
    err = oracle.rel_frobenius(got, oracle.gemm_rows(a, b, c, alpha, beta))
    del b
    ms = sum(times) / len(times)
    shape, grid = pl.super_shape(2)
    return {"ms_per_step": ms, "tflops": gemm_flops(MNK, MNK, MNK) / (ms * 1e-3) / 1e12,
            "path": "job text -> phobos_plan_make (HomeLoadPeerFetch) -> one executor per GPU; A, B, C device-resident, "
                    "each whole on one GPU (" + ", ".join(str(h) for h in homes) + "); timed on the device per "
                    "executor, the longest counts",
            "run_ms": [round(t, 3) for t in times], "warmup_runs": warm, "per_node_ms_last_run": per_node, "supertile": list(shape), "output_grid": list(grid), "supers": supers,
            "predicted_ms": (ranked[0]["makespan_sec"] * 1e3) if ranked else None, "fetch_bytes_planned": pl.fetch_bytes,
            "fetch_bytes_served": served, "fetch_matches_plan": served == pl.fetch_bytes,
            "parity": {"rel_frobenius": err, "tol": 1e-5, "rows": int(rows.size), "ok": bool(err <= 1e-5)}}


def fill_block(ph, t, seed, row0, col0, pitch):
    """Fills t[r, c] with element (row0 + r) * pitch + col0 + c of the Lcg stream `seed`."""
    ph.fill_random_block(t, seed=seed, first=row0 * pitch + col0, stream_pitch=pitch)


# ---------------------------------------------------------------------------------------------
def run_reference(args, world, rank):
    """The reference's CPU arithmetic for the workload, on the host cores (rank 0 only)."""
    if rank != 0:
        return
    import __graft_entry__ as entry  # noqa: F401  (oracle only; the product library is not loaded)
    import oracle
    oracle.build()
    oracle.use_all_cores()      # under torchrun the workers inherit OMP_NUM_THREADS=1; the other ranks have exited
    # the workload of this arm at every N: the headline GEMM (at N > 1 the GPU arm runs it as N replicas;
    # the host has one set of cores, so its rate is the same figure)
    name, M, N, K, alpha, beta = "gemm_fp16tc_fp32acc", 4096, 4096, 4096, 1.0, 0.0
    vals = []
    sample = ""
    for i in range(args.warmup + args.steps):
        r = cpu_gemm_baseline(name, M, N, K, alpha, beta, budget_flops=1.5e11, min_seconds=5.0)
        if i >= args.warmup:
            vals.append(r["value"])
        sample = r["sample"]
    v = sum(vals) / len(vals)
    fl_full = gemm_flops(M, N, K)
    line = {"impl": "reference", "metric": "GEMM & flash-attn TFLOP/s at 1/2/4/8 B200 and % of dtype roofline",
            "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": fl_full / (v * 1e12) * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64",
            "data": "synthetic (seeded Lcg, phobos-base/src/rng.rs)",
            "config": {"workload": name, "M": M, "N": N, "K": K, "alpha": alpha, "beta": beta,
                       "note": "ms_per_step extrapolates the sampled rows to the full problem"},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-suite", action="store_true", help="headline workload only")
    ap.add_argument("--only", "--bench", dest="only", default=None,
                    help="run one workload as the headline (the reference bench's --bench NAME)")
    ap.add_argument("--csv", nargs="?", const="results.csv", default=None,
                    help="also write the reference bench's CSV (phobos-bench/src/report.rs:71-88) to PATH")
    ap.add_argument("--peak-fp32", type=float, default=None, help="TFLOP/s; overrides the fp32 peak of the CSV")
    ap.add_argument("--peak-fp16tc", type=float, default=None, help="TFLOP/s; overrides the f16-tc peak of the CSV")
    ap.add_argument("--peak-fp16tcf32acc", type=float, default=None,
                    help="TFLOP/s; overrides the f16-tc-f32-acc peak of the CSV")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--kernel-only", action="store_true",
                    help="with --only: just the timed launches of the workload (no CPU baseline, end-to-end leg, parity "
                         "check or cuBLAS bar); the command the ncu captures under profiles/ are taken with")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import __graft_entry__ as entry
    ph = entry.load_package()
    ph.lib()  # no fallback: raises if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the leaf kernels have no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks = load_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ctx = Ctx(ph, torch, dev, args.steps, args.warmup)
    metric = "GEMM & flash-attn TFLOP/s at 1/2/4/8 B200 and % of dtype roofline"
    cpu = not args.no_cpu
    if args.kernel_only:
        if not args.only:
            raise SystemExit("--kernel-only needs --only WORKLOAD")
        cpu = False
        ctx.lean = True

    if world > 1 or args.gpus > 1:
        import torch.distributed as dist
        if world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        # (1) the headline workload as N independent replicas, one per GPU: no exchange, weak scaling
        ctx.barrier = dist.barrier
        head = bench_gemm(ctx, "gemm_fp16tc_fp32acc", 4096, 4096, 4096, 1.0, 0.0, peaks, cpu_baseline=False, bar=False)
        t = torch.tensor([head["ms_per_step"], head["e2e"]["ms_per_step"], head["parity"]["rel_frobenius"]], device=dev,
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_head, ms_head_e2e, head_err = (float(x) for x in t.tolist())
        head["parity"]["rel_frobenius"] = head_err           # the worst replica
        head["parity"]["ok"] = bool(head_err <= head["parity"]["tol"])
        fl = gemm_flops(4096, 4096, 4096)
        # (2) the one configuration that is partitioned across GPUs: matmul_cluster_fp32 16384^3, strong scaling
        ctx.barrier = None
        res = bench_partitioned(ctx, world, rank, 16384, 0.125, 1.5)
        torch.cuda.empty_cache()
        # (3) the same problem through the C ABI alone: rank 0 drives one executor per GPU; the other ranks wait on
        # the host (a key in the rendezvous store), so that no collective kernel sits on their GPUs meanwhile
        store = dist.distributed_c10d._get_default_store()
        plan_res = None
        if rank == 0:
            try:
                plan_res = bench_plan_driven(ctx, world, 16384, 0.125, 1.5)
            finally:
                store.set("phobos_plan_driven_done", "1")
        else:
            store.wait(["phobos_plan_driven_done"])
        dist.barrier()
        if rank == 0:
            line = {"metric": metric, "value": world * fl / (ms_head * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                    "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_head,
                    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 x f16 -> f32",
                    "data": "synthetic (seeded Lcg streams of phobos-base/src/rng.rs, generated on the device)",
                    "config": {"workload": "gemm_fp16tc_fp32acc", "M": 4096, "N": 4096, "K": 4096, "alpha": 1.0, "beta": 0.0,
                               "parallelism": f"{world} independent replicas, one per GPU (the single-GPU leaves do not "
                               "shard: replicas only); the partitioned configuration is under \"partitioned\"",
                               "l2": f"{head.get('input_sets', 1)} rotating input sets, working set larger than L2"},
                    "roofline": head["roofline"], "cpu_baseline": None,
                    "e2e": {"value": world * fl / (ms_head_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_head_e2e,
                            "h2d_bytes_per_step": world * head["e2e"]["h2d_bytes_per_step"],
                            "d2h_bytes_per_step": world * head["e2e"]["d2h_bytes_per_step"]},
                    "gpu_launches": args.steps * world,
                    "parity": head.get("parity")}
            detail = {"workload": "matmul_cluster_fp32", "M": 16384, "N": 16384, "K": 16384, "alpha": 0.125, "beta": 1.5,
                      "dtype": "f32",
                      "parallelism": f"2-D C partition {res['grid']}, K chunks of {res['k_chunk']}"
                      " copied over NVLink one step ahead of the step leaf ("
                      + ("peer copies out of the home ranks' shards, no collective" if res["exchange"] == "p2p"
                         else "NCCL broadcast") + ")",
                      "roofline": res["roofline"], "e2e": {k: v for k, v in res["e2e"].items()},
                      "gpu_launches": res["gpu_launches"], "peer_bytes_per_step": res["peer_bytes_per_step"],
                      "direct_load_bound": res["direct_load_bound"], "plan_driven": plan_res}
            # the compact summary goes last so that it survives a truncated tail of this line
            summary = {"workload": "matmul_cluster_fp32 16384^3", "scaling": "strong", "value": round(res["tflops"], 2),
                       "unit": "TFLOP/s", "ms_per_step": round(res["ms_per_step"], 3), "grid": res["grid"],
                       "exchange": res["exchange"], "one_gpu_ms_per_step": round(res["one_gpu_ms_per_step"], 3),
                       "efficiency": round(res["efficiency"], 4),
                       "zero_exchange_bound_tflops": round(res["direct_load_bound"]["tflops"], 2),
                       "frac_fp32_peak": round(res["roofline"]["frac"], 4), "parity": res["parity"]}
            if plan_res:
                summary["plan_driven_c_abi"] = {"tflops": round(plan_res["tflops"], 2), "ms_per_step": round(plan_res["ms_per_step"], 3),
                                                "vs_python_orchestrated": round(plan_res["tflops"] / res["tflops"], 4),
                                                "fetch_matches_plan": plan_res["fetch_matches_plan"],
                                                "parity_ok": plan_res["parity"]["ok"]}
        dist.barrier()
        sampler.stop()
        ok = res["parity"]["ok"] and head["parity"]["ok"] and (plan_res is None or plan_res["parity"]["ok"])
        if rank == 0:
            line["clocks"] = sampler.summary(ctx.windows)
            line["partitioned_detail"] = detail
            line["partitioned"] = summary
            print(json.dumps(line), flush=True)
        dist.destroy_process_group()
        if not ok:
            raise SystemExit("parity check failed: see the parity objects of the line above")
        return

    suite = {}
    runners = {
        "gemm_fp16tc_fp32acc": lambda: bench_gemm(ctx, "gemm_fp16tc_fp32acc", 4096, 4096, 4096, 1.0, 0.0, peaks, cpu),
        "gemm_fp32": lambda: bench_gemm(ctx, "gemm_fp32", 4096, 4096, 4096, 0.125, 1.5, peaks, cpu),
        "gemm_fp16": lambda: bench_gemm(ctx, "gemm_fp16", 8192, 8192, 8192, 1.0, 1.0, peaks, cpu),
        "flash_fp16": lambda: bench_flash(ctx, 128, 4096, 128, peaks, cpu),
        "flash_fp32": lambda: bench_flash(ctx, 128, 4096, 128, peaks, cpu_baseline=False, f32_storage=True),
        "matmul_cluster_fp32": lambda: bench_gemm(ctx, "matmul_cluster_fp32", 16384, 16384, 16384, 0.125, 1.5, peaks,
                                                  cpu_baseline=False, e2e=False),
        "saxpy_fp32": lambda: bench_saxpy(ctx, 1 << 25, peaks, cpu),
    }
    head_name = args.only or "gemm_fp16tc_fp32acc"
    ctx.cpu_seconds = 10.0     # the headline's CPU baseline gets a sample of about ten seconds
    head = runners[head_name]()
    ctx.cpu_seconds = 1.0
    if not args.no_suite and not args.only:
        for name, fn in runners.items():
            if name != head_name:
                steps_save = ctx.steps
                if name == "matmul_cluster_fp32":
                    ctx.steps = min(ctx.steps, 5)
                suite[name] = fn()
                ctx.steps = steps_save
    sampler.stop()
    results = {head_name: head, **suite}

    def target_entry(r, what):
        """The few figures of one workload that the targets are judged on, short enough to survive a cut tail."""
        rf = r["roofline"]
        e = {"tflops": round(r["tflops"], 1)}
        if rf["bound"] == "tensor":
            e["frac_nominal"] = round(rf["frac_of_nominal_2250"], 4)
            e["frac_measured"] = round(rf["frac"], 4)
        else:
            e["frac_fp32_peak"] = round(rf["frac"], 4)
        if "frac_per_clock" in rf:
            e["frac_per_clock"] = round(rf["frac_per_clock"], 4)
            e["sm_mhz"] = rf["sm_mhz_in_launch"]
        if "same_box_bar" in r:
            e["cublas_tflops"] = round(r["same_box_bar"]["tflops"], 1)
        pr = r.get("parity")
        if pr:
            e["parity"] = {"err": float(f"{pr['rel_frobenius']:.3g}"), "tol": pr["tol"], "ok": pr["ok"]}
        if what:
            e["target"] = what
        return e

    wanted = (("gemm_fp16", "gemm_fp16_8192", ">=0.70 nominal"), ("flash_fp16", "flash_fp16", ">=0.60 nominal"),
              ("gemm_fp16tc_fp32acc", "gemm_fp16tc_fp32acc_4096", None), ("gemm_fp32", "gemm_fp32_4096", None),
              ("matmul_cluster_fp32", "matmul_cluster_fp32_16384_1gpu", None))
    targets = {key: target_entry(results[name], what) for name, key, what in wanted if name in results}
    all_ok = all(r.get("parity", {"ok": True})["ok"] for r in results.values())
    # bulky per-workload records first, the compact targets last (a truncated tail of the line keeps them)
    for r in suite.values():
        cb = r.get("cpu_baseline")
        if cb:
            cb.pop("sample", None)
    line = {"metric": metric, "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": {"gemm_fp32": "f32", "matmul_cluster_fp32": "f32", "gemm_fp16": "f16", "saxpy_fp32": "f32"}.get(head_name, "f16 x f16 -> f32"),
            "data": "synthetic (seeded Lcg streams of phobos-base/src/rng.rs, generated on the device)",
            "config": {"workload": head_name, **{k: head[k] for k in head if k in ("M", "N", "K", "n", "alpha", "beta", "batch_heads", "seq_len", "head_dim")},
                       "l2": f"{head.get('input_sets', 1)} rotating input sets, working set larger than L2"},
            "roofline": head["roofline"], "cpu_baseline": head.get("cpu_baseline"), "e2e": head.get("e2e"),
            "gpu_launches": args.steps * head.get("launches_per_step", 1), "parity": head.get("parity"), "same_box_bar": head.get("same_box_bar"),
            "clocks": sampler.summary(ctx.windows), "suite": suite, "targets": targets}
    if args.csv:
        write_csv(args.csv, results, args, ph.device_info(dev.index or 0))
    print(json.dumps(line), flush=True)
    if not all_ok:
        raise SystemExit("parity check failed: see the parity objects of the line above")


def write_csv(path, results, args, info):
    """The reference bench's CSV (columns and precision labels of phobos-bench/src/report.rs:18-25, 71-88), then
    this build's extra columns.  Peaks: fp32 from the device (SMs x 128 lanes x 2 x clock, report.rs:125-147);
    both tensor-core precisions at the part's dense f16 rate (B200 accumulates in f32 at full rate, unlike the
    consumer parts the reference halves); the --peak-* flags override, as in the reference."""
    peaks = {"f32": (args.peak_fp32 * 1e3) if args.peak_fp32 else info.fp32_peak_flops / 1e9,
             "f16-tc": (args.peak_fp16tc or NOMINAL_F16_TFLOPS) * 1e3,
             "f16-tc-f32-acc": (args.peak_fp16tcf32acc or NOMINAL_F16_TFLOPS) * 1e3}
    precision = {"gemm_fp32": "f32", "matmul_cluster_fp32": "f32", "saxpy_fp32": "f32", "gemm_fp16": "f16-tc",
                 "gemm_fp16tc_fp32acc": "f16-tc-f32-acc", "flash_fp16": "f16-tc-f32-acc", "flash_fp32": "f16-tc-f32-acc"}
    rows = ["benchmark,impl,precision,gflops,peak_gflops,pct_of_peak,n_gpus,ms_per_launch,roofline_bound,roofline_frac"]
    for name, r in results.items():
        prec = precision[name]
        gf = r["tflops"] * 1e3
        rows.append(f"{name},phobos-b200,{prec},{gf:.1f},{peaks[prec]:.1f},{100.0 * gf / peaks[prec]:.1f},1,"
                    f"{r['ms_per_launch']:.4f},{r['roofline']['bound']},{r['roofline']['frac']:.3f}")
        bar = r.get("same_box_bar")
        if bar:
            rows.append(f"{name},cublas,{prec},{bar['tflops'] * 1e3:.1f},{peaks[prec]:.1f},"
                        f"{100.0 * bar['tflops'] * 1e3 / peaks[prec]:.1f},1,{bar['ms_per_step']:.4f},,")
        cb = r.get("cpu_baseline")
        if cb:
            rows.append(f"{name},cpu-{cb['kind']},f64,{cb['value'] * 1e3:.1f},,,0,,,")
    Path(path).write_text("\n".join(rows) + "\n")


if __name__ == "__main__":
    main()
