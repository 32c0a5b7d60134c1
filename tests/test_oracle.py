"""The CPU oracle against the golden fixtures (tests/golden/, made by make_golden.py through an
independent pure-Python route) and against its own cross-checks.  No GPU."""
import json
from pathlib import Path

import numpy as np
import pytest

G = Path(__file__).resolve().parent / "golden"


def _load(name):
    return json.loads((G / name).read_text())


def test_lcg_matches_hand_rolled_recurrence(oracle):
    """phobos-base/src/rng.rs:51-63."""
    g = _load("lcg.json")
    for seed in ("1", "2", "42"):
        assert [str(s) for s in oracle.lcg_u64(int(seed), 16)] == g[seed]["states"]
        got = oracle.lcg_fill(int(seed), 16).view(np.uint32).tolist()
        assert got == g[seed]["unit_bits"]


def test_lcg_skip_ahead_and_threads(oracle):
    g = _load("lcg.json")["skip"]
    big = oracle.lcg_fill(g["seed"], g["index"] + 1)   # filled by several threads with skip-ahead
    assert int(big[-1:].view(np.uint32)[0]) == g["unit_bits"]
    assert np.array_equal(big[:16], oracle.lcg_fill(g["seed"], 16))
    assert (big >= -1.0).all() and (big < 1.0).all()          # rng.rs:43-49
    assert not np.array_equal(oracle.lcg_fill(1, 16), oracle.lcg_fill(2, 16))   # rng.rs:37-40


def test_f16_rounding_is_ieee_rn_even(oracle):
    g = _load("f16.json")
    x = np.array(g["f32_bits"], dtype=np.uint32).view(np.float32)
    assert oracle.f32_to_f16_bits(x).tolist() == g["f16_bits"]
    rng = np.random.default_rng(0)
    y = (rng.standard_normal(1 << 16) * 10.0 ** rng.integers(-9, 5, 1 << 16)).astype(np.float32)
    assert np.array_equal(oracle.f32_to_f16_bits(y), y.astype(np.float16).view(np.uint16))
    allh = np.arange(65536, dtype=np.uint16)
    f = oracle.f16_bits_to_f32(allh)
    ref = allh.view(np.float16).astype(np.float32)
    assert np.array_equal(f.view(np.uint32), ref.view(np.uint32))


def test_sample_points_match_the_verifier(oracle):
    """phobos-bench/src/main.rs:403-416."""
    g = _load("samples.json")
    for key, want in g.items():
        r, c = (int(v) for v in key.split("x"))
        assert oracle.sample_points(r, c).tolist() == want


def test_gemm_oracle_exact_integer_case(oracle):
    """phobos-bench/examples/masking.rs:109-147."""
    g = _load("masking.json")
    M, K, N = g["M"], g["K"], g["N"]
    a = ((np.arange(M * K) % 7) - 3).astype(np.float32).reshape(M, K)
    b = ((np.arange(K * N) % 5) - 2).astype(np.float32).reshape(K, N)
    c = np.zeros((M, N), dtype=np.float32)
    out = oracle.gemm_rows(a, b, c, 1.0, 0.0)
    assert out.sum(axis=1).tolist() == g["row_sums"]
    assert out.sum(axis=0).tolist() == g["col_sums"]
    assert [out[0, 0], out[0, -1], out[-1, 0], out[-1, -1]] == g["corners"]
    assert np.abs(out).sum() == g["abs_sum"]


def test_gemm_oracle_against_numpy_f64(oracle):
    M, N, K = 70, 52, 300      # ragged against the oracle's blocking
    a = oracle.lcg_fill(1, M * K).reshape(M, K)
    b = oracle.lcg_fill(2, K * N).reshape(K, N)
    c = oracle.lcg_fill(3, M * N).reshape(M, N)
    want = 0.125 * (a.astype(np.float64) @ b.astype(np.float64)) + 1.5 * c.astype(np.float64)
    assert np.allclose(oracle.gemm_rows(a, b, c, 0.125, 1.5), want, rtol=0, atol=1e-12)
    rows = np.array([3, 69, 0, 17], dtype=np.uint64)
    assert np.allclose(oracle.gemm_rows(a, b, c, 0.125, 1.5, rows=rows), want[rows.astype(int)], atol=1e-12)
    a16, b16 = a.astype(np.float16).astype(np.float64), b.astype(np.float16).astype(np.float64)
    want16 = a16 @ b16
    got16 = oracle.gemm_rows(a, b, c, 1.0, 0.0, round_inputs_f16=True)
    assert np.allclose(got16, want16, atol=1e-12)


def test_f16_sequential_accumulate_model(oracle):
    """phobos-bench/src/main.rs:663-670, restated here in numpy float16/float32 steps."""
    N, K = 8, 200
    a = oracle.fp16_round(oracle.lcg_fill(5, 4 * K).reshape(4, K))
    b = oracle.fp16_round(oracle.lcg_fill(6, K * N).reshape(K, N))
    c = oracle.fp16_round(oracle.lcg_fill(7, 4 * N).reshape(4, N))
    pts = np.array([[0, 0], [3, 7], [2, 5]], dtype=np.uint64)
    got = oracle.gemm_f16acc_points(a, b, c, 1.0, 1.0, pts)
    for (i, j), g in zip(pts.astype(int), got):
        acc = np.float32(0)
        for k in range(K):
            acc = np.float32(np.float16(np.float32(acc + np.float32(a[i, k] * b[k, j]))))
        want = np.float32(np.float16(np.float32(np.float32(1.0) * acc + np.float32(1.0) * c[i, j])))
        assert g == want


def test_flash_oracle_against_two_pass_softmax(oracle):
    g = _load("flash.json")
    Nq, Nk, D = g["Nq"], g["Nk"], g["D"]
    q = oracle.fp16_round(oracle.lcg_fill(g["seeds"][0], Nq * D)).reshape(Nq, D)
    k = oracle.fp16_round(oracle.lcg_fill(g["seeds"][1], Nk * D)).reshape(Nk, D)
    v = oracle.fp16_round(oracle.lcg_fill(g["seeds"][2], Nk * D)).reshape(Nk, D)
    out = oracle.flash_rows(q, k, v, g["scale"])
    assert np.allclose(out, np.array(g["out"]), rtol=0, atol=1e-13)
    rows = np.array([5, 0, 15], dtype=np.uint64)
    assert np.allclose(oracle.flash_rows(q, k, v, g["scale"], rows=rows), np.array(g["out"])[rows.astype(int)], atol=1e-13)


def test_error_measures(oracle):
    want = np.array([3.0, 4.0, 0.0])
    got = np.array([3.0, 4.0, 0.5], dtype=np.float32)
    assert oracle.rel_frobenius(got, want) == pytest.approx(0.1)
    assert oracle.max_rel_floor(got, want, 0.1) == pytest.approx(5.0)
    assert oracle.max_rel_floor(got, want, 1.0) == pytest.approx(0.5)


def test_normal_generator_statistics(oracle):
    x = oracle.lcg_fill_normal(4, 1 << 18)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01
    assert np.array_equal(x[:101], oracle.lcg_fill_normal(4, 101))


def test_saxpy_rounds_the_product_then_the_sum(oracle):
    """verify_saxpy (phobos-bench/src/main.rs:1179-1188) against numpy's separately rounded f32 ops."""
    x, y = oracle.lcg_fill(42, 100003), oracle.lcg_fill(43, 100003)
    for alpha in (2.0, 0.3, -1.7):
        want = (np.float32(alpha) * x) + y              # numpy rounds each f32 operation
        assert np.array_equal(oracle.saxpy(x, y, alpha).view(np.uint32), want.view(np.uint32))


def test_kda_chunked_form_equals_the_recurrence(oracle):
    """The chunked evaluation the kernel body spells out (cumsum / tril / carried state) is the token-by-token
    recurrence S_t = a_t S_{t-1} + k_t^T v_t, o_t = scale q_t S_t of its header (examples/kda_fp32.ph:3-18),
    for any chunk size, ragged tails included."""
    n, d = 200, 64
    q, k, v = (oracle.lcg_fill(s, n * d).reshape(n, d) for s in (7, 8, 9))
    g = -np.abs(oracle.lcg_fill(10, n)) * 0.2            # log forget-gates, <= 0
    want = oracle.kda(q, k, v, g, 0.125)
    assert np.abs(want).max() > 0.1
    for chunk in (1, 32, 64, 128, 200):
        got = oracle.kda(q, k, v, g, 0.125, chunk=chunk)
        assert np.abs(got - want).max() <= 1e-12 * max(1.0, np.abs(want).max())
    # a known answer: gates of zero (a_t = 1) and orthonormal keys make S a plain sum of outer products
    e = np.eye(4, 64, dtype=np.float32)
    vv = np.arange(4 * 64, dtype=np.float32).reshape(4, 64)
    out = oracle.kda(e, e, vv, np.zeros(4, np.float32), 1.0)
    assert np.array_equal(out, vv.astype(np.float64))     # o_t = q_t S_t = v_t
