"""ctypes front end of the CPU oracle (``oracle/phobos_oracle.c``).

TEST INFRASTRUCTURE ONLY.  The product package never imports this module; it
exists so that tests, the smoke check and the benchmark's CPU-baseline leg can
compare the CUDA kernels with a CPU restatement of the reference's own
verifier arithmetic (phobos-bench/src/main.rs:386-445, 638-679, 869-920) on
inputs from the reference's in-tree generator (phobos-base/src/rng.rs:1-26).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libphobos_oracle.so"
_lib = None

_u64p = ctypes.POINTER(ctypes.c_uint64)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(force: bool = False) -> Path:
    """Compile the oracle with the system gcc (see oracle/Makefile)."""
    src = _HERE / "phobos_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(_HERE), "-B", "libphobos_oracle.so"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_SO))
        L.ph_oracle_lcg_next_u64.restype = ctypes.c_uint64
        L.ph_oracle_lcg_next_u64.argtypes = [_u64p]
        L.ph_oracle_lcg_fill.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _f32p]
        L.ph_oracle_lcg_fill_normal.argtypes = [ctypes.c_uint64, ctypes.c_uint64, _f32p]
        L.ph_oracle_lcg_fill_normal_at.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, _f32p]
        L.ph_oracle_lcg_fill_block.argtypes = [ctypes.c_uint64] * 5 + [ctypes.c_float, _f32p]
        L.ph_oracle_f32_to_f16_bits.argtypes = [_f32p, ctypes.c_uint64, _u16p]
        L.ph_oracle_f16_bits_to_f32.argtypes = [_u16p, ctypes.c_uint64, _f32p]
        L.ph_oracle_sample_points.argtypes = [ctypes.c_uint64, ctypes.c_uint64, _u64p]
        L.ph_oracle_gemm_rows.restype = ctypes.c_int
        L.ph_oracle_gemm_rows.argtypes = [ctypes.c_uint64] * 3 + [_f32p, _f32p, _f32p, ctypes.c_double,
                                                                  ctypes.c_double, ctypes.c_int, _u64p,
                                                                  ctypes.c_uint64, _f64p]
        L.ph_oracle_gemm_f16acc_points.argtypes = [ctypes.c_uint64, ctypes.c_uint64, _f32p, _f32p, _f32p,
                                                   ctypes.c_float, ctypes.c_float, _u64p, ctypes.c_uint64,
                                                   _f32p]
        L.ph_oracle_flash_rows.restype = ctypes.c_int
        L.ph_oracle_flash_rows.argtypes = [ctypes.c_uint64] * 3 + [_f32p, _f32p, _f32p, ctypes.c_double, _u64p,
                                                                   ctypes.c_uint64, _f64p]
        for fn, extra in ((L.ph_oracle_kda_recurrence, []), (L.ph_oracle_kda_chunked, [ctypes.c_uint64])):
            fn.restype = None
            fn.argtypes = [_f32p, _f32p, _f32p, _f32p, ctypes.c_uint64, ctypes.c_uint64] + extra + [ctypes.c_double, _f64p]
        L.ph_oracle_saxpy.restype = None
        L.ph_oracle_saxpy.argtypes = [_f32p, _f32p, ctypes.c_float, ctypes.c_uint64, _f32p]
        L.ph_oracle_rel_frobenius.restype = ctypes.c_double
        L.ph_oracle_rel_frobenius.argtypes = [_f32p, _f64p, ctypes.c_uint64]
        L.ph_oracle_max_rel_floor.restype = ctypes.c_double
        L.ph_oracle_max_rel_floor.argtypes = [_f32p, _f64p, ctypes.c_uint64, ctypes.c_double]
        L.ph_oracle_threads.restype = ctypes.c_int
        L.ph_oracle_set_threads.restype = None
        L.ph_oracle_set_threads.argtypes = [ctypes.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def threads() -> int:
    return int(lib().ph_oracle_threads())


def use_all_cores() -> int:
    """Sets the OpenMP thread count to the cores this process may run on (a launcher such as torchrun
    exports OMP_NUM_THREADS=1 to its workers) and returns it."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().ph_oracle_set_threads(n)
    return threads()


def lcg_u64(seed: int, n: int) -> list[int]:
    """First ``n`` raw states of Lcg::new(seed) (rng.rs:9-15)."""
    s = ctypes.c_uint64(seed)
    return [int(lib().ph_oracle_lcg_next_u64(ctypes.byref(s))) for _ in range(n)]


def lcg_fill(seed: int, n: int, scale: float = 1.0) -> np.ndarray:
    """``scale * Lcg::new(seed).unit_f32s(n)`` (rng.rs:17-25)."""
    out = np.empty(n, dtype=np.float32)
    lib().ph_oracle_lcg_fill(seed, n, scale, _p(out, _f32p))
    return out


def lcg_fill_block(seed: int, first: int, rows: int, cols: int, pitch: int, scale: float = 1.0) -> np.ndarray:
    """A [rows, cols] block of a larger seeded tensor: element (r, c) is stream element first + r*pitch + c."""
    out = np.empty((rows, cols), dtype=np.float32)
    lib().ph_oracle_lcg_fill_block(seed, first, rows, cols, pitch, scale, _p(out, _f32p))
    return out


def lcg_fill_normal(seed: int, n: int, first: int = 0) -> np.ndarray:
    """N(0,1) by Box-Muller over the Lcg stream, from element `first` (even) on."""
    assert first % 2 == 0
    out = np.empty(n, dtype=np.float32)
    lib().ph_oracle_lcg_fill_normal_at(seed, first, n, _p(out, _f32p))
    return out


def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x).ravel()
    out = np.empty(x.size, dtype=np.uint16)
    lib().ph_oracle_f32_to_f16_bits(_p(x, _f32p), x.size, _p(out, _u16p))
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16).ravel()
    out = np.empty(h.size, dtype=np.float32)
    lib().ph_oracle_f16_bits_to_f32(_p(h, _u16p), h.size, _p(out, _f32p))
    return out


def fp16_round(x) -> np.ndarray:
    """f32 -> f16 -> f32 (main.rs:447-449)."""
    x = _f32(x)
    return f16_bits_to_f32(f32_to_f16_bits(x)).reshape(x.shape)


def sample_points(rows: int, cols: int) -> np.ndarray:
    """The verifier's 64 (i, j) positions (main.rs:403-416)."""
    out = np.empty((64, 2), dtype=np.uint64)
    lib().ph_oracle_sample_points(rows, cols, _p(out, _u64p))
    return out


def gemm_rows(a, b, c_in, alpha, beta, rows=None, round_inputs_f16=False) -> np.ndarray:
    """f64 ``alpha * a@b + beta * c_in`` for the given rows (all if None)."""
    a, b, c_in = _f32(a), _f32(b), _f32(c_in)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2 and c_in.shape == (M, N)
    rows = np.arange(M, dtype=np.uint64) if rows is None else np.ascontiguousarray(rows, dtype=np.uint64)
    out = np.empty((rows.size, N), dtype=np.float64)
    rc = lib().ph_oracle_gemm_rows(M, N, K, _p(a, _f32p), _p(b, _f32p), _p(c_in, _f32p), float(alpha),
                                   float(beta), int(round_inputs_f16), _p(rows, _u64p), rows.size,
                                   _p(out, _f64p))
    if rc != 0:
        raise MemoryError("oracle gemm")
    return out


def gemm_f16acc_points(a, b, c_in, alpha, beta, points) -> np.ndarray:
    """The reference's sequential f16-accumulate model at (i, j) points (main.rs:663-670)."""
    a, b, c_in = _f32(a), _f32(b), _f32(c_in)
    K, N = b.shape
    pts = np.ascontiguousarray(points, dtype=np.uint64)
    out = np.empty(pts.shape[0], dtype=np.float32)
    lib().ph_oracle_gemm_f16acc_points(N, K, _p(a, _f32p), _p(b, _f32p), _p(c_in, _f32p), float(alpha),
                                       float(beta), _p(pts, _u64p), pts.shape[0], _p(out, _f32p))
    return out


def flash_rows(q, k, v, scale, rows=None) -> np.ndarray:
    """f64 online-softmax attention for the given query rows of one head (main.rs:894-911)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    Nq, D = q.shape
    Nk = k.shape[0]
    assert k.shape == (Nk, D) and v.shape == (Nk, D)
    rows = np.arange(Nq, dtype=np.uint64) if rows is None else np.ascontiguousarray(rows, dtype=np.uint64)
    out = np.empty((rows.size, D), dtype=np.float64)
    rc = lib().ph_oracle_flash_rows(Nq, Nk, D, _p(q, _f32p), _p(k, _f32p), _p(v, _f32p), float(scale),
                                    _p(rows, _u64p), rows.size, _p(out, _f64p))
    if rc != 0:
        raise MemoryError("oracle flash")
    return out


def kda(q, k, v, g, scale: float, chunk: int | None = None) -> np.ndarray:
    """Gated linear attention of one head in f64 (examples/kda_fp32.ph): token by token when `chunk` is None
    (the recurrence the kernel's header states), else chunk by chunk the way the kernel body is written."""
    q, k, v = (_f32(x) for x in (q, k, v))
    g = _f32(g).ravel()
    n, d = q.shape
    assert k.shape == (n, d) and v.shape == (n, d) and g.size == n
    out = np.empty((n, d), dtype=np.float64)
    if chunk is None:
        lib().ph_oracle_kda_recurrence(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), _p(g, _f32p), n, d, scale, _p(out, _f64p))
    else:
        lib().ph_oracle_kda_chunked(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), _p(g, _f32p), n, d, chunk, scale,
                                    _p(out, _f64p))
    return out


def saxpy(x, y, alpha: float) -> np.ndarray:
    """alpha * x + y in f32, product and sum rounded separately (verify_saxpy, main.rs:1179-1188)."""
    x, y = _f32(x).ravel(), _f32(y).ravel()
    assert x.size == y.size
    out = np.empty(x.size, dtype=np.float32)
    lib().ph_oracle_saxpy(_p(x, _f32p), _p(y, _f32p), alpha, x.size, _p(out, _f32p))
    return out


def rel_frobenius(got, want) -> float:
    got = _f32(got).ravel()
    want = np.ascontiguousarray(want, dtype=np.float64).ravel()
    assert got.size == want.size
    return float(lib().ph_oracle_rel_frobenius(_p(got, _f32p), _p(want, _f64p), got.size))


def max_rel_floor(got, want, floor: float) -> float:
    got = _f32(got).ravel()
    want = np.ascontiguousarray(want, dtype=np.float64).ravel()
    assert got.size == want.size
    return float(lib().ph_oracle_max_rel_floor(_p(got, _f32p), _p(want, _f64p), got.size, floor))
