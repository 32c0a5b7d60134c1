/*
 * CPU oracle for the phobos leaf kernels.  TEST INFRASTRUCTURE ONLY: nothing
 * the product ships may link, load or call this file.  It restates, in plain
 * C, the reference's own host-side arithmetic for the leaf kernels (its f64
 * verifier functions and its input generator).  Every function cites the
 * reference lines it follows (paths relative to the phobos repository root).
 *
 * Pinning: the reference stores no golden vectors and cannot be built where
 * this oracle was written (it is Rust + LLVM/MLIR).  The oracle is pinned
 * against the known-answer cases the reference's own tests restate:
 *   - the Lcg recurrence guard   (phobos-base/src/rng.rs:51-63)
 *   - the exact-integer matmul   (phobos-bench/examples/masking.rs:109-147)
 *   - IEEE round-to-nearest-even f32->f16 (crate half 2.7.1, called at
 *     phobos-bench/src/main.rs:447-449), checked against numpy.float16
 *   - an independent two-pass softmax for the flash recurrence
 * The bench input streams of the reference come from rand 0.8.6 SmallRng
 * (phobos-bench/src/main.rs:472), a third-party crate that is not vendored:
 * for those streams parity is unpinned, and the in-tree Lcg is used instead.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define PH_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* Lcg: phobos-base/src/rng.rs:9-20                                    */
/* ------------------------------------------------------------------ */
#define LCG_A 6364136223846793005ULL
#define LCG_C 1442695040888963407ULL

static inline uint64_t lcg_next(uint64_t *s) {
  *s = *s * LCG_A + LCG_C; /* wrapping mod 2^64: rng.rs:10-15 */
  return *s;
}

/* (state >> 33) as f32 / 2^31 - 1.0 : rng.rs:18-20.  The u64->f32 cast of a
 * 31-bit integer rounds to nearest-even exactly as C's (float) does. */
static inline float lcg_unit(uint64_t *s) {
  return (float)(lcg_next(s) >> 33) / (float)(1ULL << 31) - 1.0f;
}

/* Jump `n` steps ahead: x -> A^n x + C (A^n - 1)/(A - 1), by square and
 * multiply on the affine map.  Only used to split one stream over threads;
 * the values are those of the sequential recurrence. */
static uint64_t lcg_skip(uint64_t s, uint64_t n) {
  uint64_t a = LCG_A, c = LCG_C, acc_a = 1, acc_c = 0;
  while (n) {
    if (n & 1) {
      acc_a = acc_a * a;
      acc_c = acc_c * a + c;
    }
    c = (a + 1) * c;
    a = a * a;
    n >>= 1;
  }
  return acc_a * s + acc_c;
}

PH_EXPORT uint64_t ph_oracle_lcg_next_u64(uint64_t *state) { return lcg_next(state); }

/* out[i] = scale * next_unit_f32(); scale = 1 gives Lcg::unit_f32s
 * (rng.rs:23-25), which is also `phobos-tensor init --fill random`
 * (phobos-cluster/src/bin/phobos-tensor.rs:55-72). */
PH_EXPORT void ph_oracle_lcg_fill(uint64_t seed, uint64_t n, float scale, float *out) {
#pragma omp parallel
  {
#ifdef _OPENMP
    int nt = omp_get_num_threads(), t = omp_get_thread_num();
#else
    int nt = 1, t = 0;
#endif
    uint64_t lo = n * (uint64_t)t / (uint64_t)nt, hi = n * (uint64_t)(t + 1) / (uint64_t)nt;
    uint64_t s = lcg_skip(seed, lo);
    for (uint64_t i = lo; i < hi; i++) out[i] = scale * lcg_unit(&s);
  }
}

/* Rows [0, rows) x columns [0, cols) of a block of a larger seeded tensor: out[r][c] is
 * stream element first + r*pitch + c (scaled).  This is how a rank reads its shard of a
 * tensor that `phobos-tensor init --fill random` wrote as one stream
 * (phobos-cluster/src/bin/phobos-tensor.rs:55-72, row-major, storage.rs:22-46). */
PH_EXPORT void ph_oracle_lcg_fill_block(uint64_t seed, uint64_t first, uint64_t rows, uint64_t cols, uint64_t pitch,
                                        float scale, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; r++) {
    uint64_t s = lcg_skip(seed, first + (uint64_t)r * pitch);
    float *o = out + (uint64_t)r * cols;
    for (uint64_t c = 0; c < cols; c++) o[c] = scale * lcg_unit(&s);
  }
}

/* N(0,1) by Box-Muller over consecutive Lcg pairs.  The reference has no
 * normal generator; this exists because the flash_fp16 benchmark config asks
 * for N(0,1) inputs.  u1 = (unit+1)/2 mapped into (0,1], u2 likewise. */
PH_EXPORT void ph_oracle_lcg_fill_normal_at(uint64_t seed, uint64_t first, uint64_t n, float *out);
PH_EXPORT void ph_oracle_lcg_fill_normal(uint64_t seed, uint64_t n, float *out) {
  ph_oracle_lcg_fill_normal_at(seed, 0, n, out);
}
/* The same stream from element `first` on (first must be even: elements come in pairs). */
PH_EXPORT void ph_oracle_lcg_fill_normal_at(uint64_t seed, uint64_t first, uint64_t n, float *out) {
  uint64_t pairs = (n + 1) / 2;
  seed = lcg_skip(seed, first);
#pragma omp parallel
  {
#ifdef _OPENMP
    int nt = omp_get_num_threads(), t = omp_get_thread_num();
#else
    int nt = 1, t = 0;
#endif
    uint64_t lo = pairs * (uint64_t)t / (uint64_t)nt, hi = pairs * (uint64_t)(t + 1) / (uint64_t)nt;
    uint64_t s = lcg_skip(seed, 2 * lo);
    for (uint64_t p = lo; p < hi; p++) {
      double u1 = ((double)(lcg_next(&s) >> 33) + 1.0) / 2147483648.0; /* (0,1] */
      double u2 = (double)(lcg_next(&s) >> 33) / 2147483648.0;         /* [0,1) */
      double r = sqrt(-2.0 * log(u1)), th = 6.283185307179586476925 * u2;
      out[2 * p] = (float)(r * cos(th));
      if (2 * p + 1 < n) out[2 * p + 1] = (float)(r * sin(th));
    }
  }
}

/* ------------------------------------------------------------------ */
/* f32 <-> f16, IEEE round-to-nearest-even (half::f16::from_f32,       */
/* phobos-bench/src/main.rs:447-449; device side arith.truncf,         */
/* phobos-lang/src/codegen/matmul.rs:2191-2231)                        */
/* ------------------------------------------------------------------ */
static inline uint16_t f32_to_f16_bits(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? (0x0200u | ((absx >> 13) & 0x3FFu)) : 0));
  if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf: >= 65520 */
  if (absx < 0x33000001u) return (uint16_t)sign;             /* <= 2^-25 rounds to zero */
  int32_t e = (int32_t)(absx >> 23) - 127;
  uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
  uint32_t shift, half_bits;
  if (e < -14) { /* subnormal half */
    shift = (uint32_t)(13 + (-14 - e));
    half_bits = 0;
  } else {
    shift = 13;
    half_bits = (uint32_t)(e + 15) << 10;
    m &= 0x7FFFFFu;
  }
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1))) q++;
  return (uint16_t)(sign | (half_bits + q)); /* carry into exponent is correct */
}

static inline float f16_bits_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, x;
  if (e == 0) {
    if (m == 0) {
      x = sign;
    } else {
      int sh = 0;
      while (!(m & 0x400u)) {
        m <<= 1;
        sh++;
      }
      x = sign | ((uint32_t)(113 - sh) << 23) | ((m & 0x3FFu) << 13);
    }
  } else if (e == 31) {
    x = sign | 0x7F800000u | (m << 13);
  } else {
    x = sign | ((e + 112) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &x, 4);
  return f;
}

static inline float fp16_round(float f) { return f16_bits_to_f32(f32_to_f16_bits(f)); }

PH_EXPORT void ph_oracle_f32_to_f16_bits(const float *in, uint64_t n, uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < n; i++) out[i] = f32_to_f16_bits(in[i]);
}

PH_EXPORT void ph_oracle_f16_bits_to_f32(const uint16_t *in, uint64_t n, float *out) {
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < n; i++) out[i] = f16_bits_to_f32(in[i]);
}

/* ------------------------------------------------------------------ */
/* The 64 sample positions of the reference verifiers:                 */
/* phobos-bench/src/main.rs:403-416 (xorshift64 from a fixed state)    */
/* ------------------------------------------------------------------ */
PH_EXPORT void ph_oracle_sample_points(uint64_t rows, uint64_t cols, uint64_t *out_ij /* 64*2 */) {
  uint64_t state = 0x243F6A8885A308D3ULL;
  for (int s = 0; s < 64; s++) {
    uint64_t i, j;
    if (s == 0) {
      i = 0;
      j = 0;
    } else if (s == 1) {
      i = rows - 1;
      j = cols - 1;
    } else {
      state ^= state << 13;
      state ^= state >> 7;
      state ^= state << 17;
      i = state % rows;
      state ^= state << 13;
      state ^= state >> 7;
      state ^= state << 17;
      j = state % cols;
    }
    out_ij[2 * s] = i;
    out_ij[2 * s + 1] = j;
  }
}

/* ------------------------------------------------------------------ */
/* GEMM oracle: want = alpha * sum_k f64(a_ik) f64(b_kj) + beta * c_ij */
/* phobos-bench/src/main.rs:417-436 (verify_matmul), computed for      */
/* whole rows instead of 64 samples.  Inputs are the kernel's          */
/* storage-precision values widened to f32 (f16 values are exact in    */
/* f32); `round_inputs_f16` applies fp16_round first, as               */
/* main.rs:417-423 does for the tensor-core kernels whose .ph          */
/* signature is f32.  The order of the f64 additions differs from the  */
/* reference's plain k loop only in the last bits of an f64.           */
/* ------------------------------------------------------------------ */
#define GB_K 256
#define GB_N 512

/* acc[r][0..n) += sum_{kk<kn} a[r][kk] * b[kk][0..n) for 4 rows at once. */
__attribute__((target_clones("avx512f", "avx2", "default"))) static void
micro_4rows(double *restrict c0, double *restrict c1, double *restrict c2, double *restrict c3,
            const double *restrict a /* 4*GB_K, row-major */, const float *restrict b, uint64_t ldb,
            int kn, int n) {
  for (int kk = 0; kk < kn; kk++) {
    const float *restrict br = b + (uint64_t)kk * ldb;
    double a0 = a[kk], a1 = a[GB_K + kk], a2 = a[2 * GB_K + kk], a3 = a[3 * GB_K + kk];
#pragma omp simd
    for (int j = 0; j < n; j++) {
      double bv = (double)br[j];
      c0[j] += a0 * bv;
      c1[j] += a1 * bv;
      c2[j] += a2 * bv;
      c3[j] += a3 * bv;
    }
  }
}

PH_EXPORT int ph_oracle_gemm_rows(uint64_t M, uint64_t N, uint64_t K, const float *a, const float *b,
                                  const float *c_in, double alpha, double beta, int round_inputs_f16,
                                  const uint64_t *rows, uint64_t nrows, double *out /* nrows*N */) {
  (void)M;
  const float *bb = b;
  float *brounded = NULL;
  if (round_inputs_f16) {
    brounded = (float *)malloc(sizeof(float) * K * N);
    if (!brounded) return -1;
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < K * N; i++) brounded[i] = fp16_round(b[i]);
    bb = brounded;
  }
  uint64_t ngroups = (nrows + 3) / 4;
  int fail = 0;
#pragma omp parallel
  {
#ifdef _OPENMP
    int nt = omp_get_num_threads(), t = omp_get_thread_num();
#else
    int nt = 1, t = 0;
#endif
    /* each thread owns a contiguous run of 4-row groups and sweeps B once */
    uint64_t g_lo = ngroups * (uint64_t)t / (uint64_t)nt, g_hi = ngroups * (uint64_t)(t + 1) / (uint64_t)nt;
    double *scratch = (double *)malloc(sizeof(double) * (4 * GB_K + 4 * GB_N));
    if (!scratch) {
#pragma omp atomic write
      fail = 1;
    } else {
      double *apack = scratch, *dummy = scratch + 4 * GB_K;
      for (uint64_t g = g_lo; g < g_hi; g++)
        for (uint64_t r = 4 * g; r < 4 * g + 4 && r < nrows; r++)
          for (uint64_t j = 0; j < N; j++) out[r * N + j] = 0.0;
      for (uint64_t nb = 0; nb < N; nb += GB_N) {
        int n = (int)((N - nb) < GB_N ? (N - nb) : GB_N);
        for (uint64_t kb = 0; kb < K; kb += GB_K) {
          int kn = (int)((K - kb) < GB_K ? (K - kb) : GB_K);
          for (uint64_t g = g_lo; g < g_hi; g++) {
            double *cp[4];
            for (int rr = 0; rr < 4; rr++) {
              uint64_t r = 4 * g + (uint64_t)rr;
              if (r < nrows) {
                uint64_t i = rows[r];
                for (int kk = 0; kk < kn; kk++) {
                  float av = a[i * K + kb + (uint64_t)kk];
                  apack[rr * GB_K + kk] = (double)(round_inputs_f16 ? fp16_round(av) : av);
                }
                cp[rr] = out + r * N + nb;
              } else {
                for (int kk = 0; kk < kn; kk++) apack[rr * GB_K + kk] = 0.0;
                for (int j = 0; j < n; j++) dummy[rr * GB_N + j] = 0.0;
                cp[rr] = dummy + rr * GB_N;
              }
            }
            micro_4rows(cp[0], cp[1], cp[2], cp[3], apack, bb + kb * N + nb, N, kn, n);
          }
        }
      }
      for (uint64_t g = g_lo; g < g_hi; g++)
        for (uint64_t r = 4 * g; r < 4 * g + 4 && r < nrows; r++) {
          uint64_t i = rows[r];
          for (uint64_t j = 0; j < N; j++)
            out[r * N + j] = alpha * out[r * N + j] + beta * (double)c_in[i * N + j];
        }
      free(scratch);
    }
  }
  free(brounded);
  return fail ? -1 : 0;
}

/* Sequential per-step f16 accumulation model of the pure-f16 GEMM:
 * phobos-bench/src/main.rs:663-670 (verify_matmul_fp16acc).  acc is an f32
 * that is rounded to f16 after every multiply-add; the product and the add
 * are separate f32 operations (Rust `acc + af * bf`, no fusing). */
PH_EXPORT void ph_oracle_gemm_f16acc_points(uint64_t N, uint64_t K, const float *a, const float *b,
                                            const float *c_in, float alpha, float beta,
                                            const uint64_t *ij, uint64_t npoints, float *out) {
#pragma omp parallel for schedule(static)
  for (uint64_t p = 0; p < npoints; p++) {
    uint64_t i = ij[2 * p], j = ij[2 * p + 1];
    volatile float acc = 0.0f;
    for (uint64_t k = 0; k < K; k++) {
      float af = fp16_round(a[i * K + k]), bf = fp16_round(b[k * N + j]);
      volatile float prod = af * bf; /* volatile: keep mul and add unfused */
      acc = fp16_round(acc + prod);
    }
    volatile float t1 = alpha * acc, t2 = beta * c_in[i * N + j];
    out[p] = fp16_round(t1 + t2);
  }
}

/* ------------------------------------------------------------------ */
/* Flash attention oracle: f64 replay of the online-softmax recurrence */
/* over the keys, phobos-bench/src/main.rs:894-911, for every column d */
/* of the chosen query rows.  q,k,v are storage-precision values       */
/* widened to f32 (the bench hands the verifier f16-rounded inputs,    */
/* main.rs:1078-1081).  m starts at -inf as in main.rs:894.            */
/* ------------------------------------------------------------------ */
PH_EXPORT int ph_oracle_flash_rows(uint64_t Nq, uint64_t Nk, uint64_t D, const float *q, const float *k,
                                   const float *v, double scale, const uint64_t *rows, uint64_t nrows,
                                   double *out /* nrows*D */) {
  (void)Nq;
  int fail = 0;
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * D);
    if (!acc) {
#pragma omp atomic write
      fail = 1;
    }
#pragma omp for schedule(dynamic, 4)
    for (uint64_t r = 0; r < nrows; r++) {
      if (!acc) continue;
      uint64_t i = rows[r];
      double m = -INFINITY, l = 0.0;
      for (uint64_t d = 0; d < D; d++) acc[d] = 0.0;
      for (uint64_t j = 0; j < Nk; j++) {
        double score = 0.0;
        for (uint64_t e = 0; e < D; e++) score += (double)q[i * D + e] * (double)k[j * D + e];
        score *= scale;
        double mnew = m > score ? m : score;
        double corr = exp(m - mnew), p = exp(score - mnew);
        l = l * corr + p;
        for (uint64_t d = 0; d < D; d++) acc[d] = acc[d] * corr + p * (double)v[j * D + d];
        m = mnew;
      }
      for (uint64_t d = 0; d < D; d++) out[r * D + d] = acc[d] / l;
    }
    free(acc);
  }
  return fail ? -1 : 0;
}

/* ------------------------------------------------------------------ */
/* Error measures                                                      */
/* ------------------------------------------------------------------ */
/* ||got - want||_F / ||want||_F over n elements (the parity bar). */
/* Gated linear attention of one head, token by token in f64: the recurrence that
 * examples/kda_fp32.ph:3-8 states as the meaning of the kernel,
 *   S_t = a_t * S_{t-1} + k_t^T v_t,   o_t = scale * q_t @ S_t,   a_t = exp(g_t).
 * The reference has no numeric check for this kernel; this is the definition its chunked
 * form must agree with.  Q, K, V, O are [n][d] row-major f32, G is [n]. */
PH_EXPORT void ph_oracle_kda_recurrence(const float *q, const float *k, const float *v, const float *g, uint64_t n, uint64_t d,
                                       double scale, double *out) {
  double *S = (double *)calloc(d * d, sizeof(double));
  for (uint64_t t = 0; t < n; t++) {
    const double a = exp((double)g[t]);
    for (uint64_t i = 0; i < d; i++) {
      const double ki = (double)k[t * d + i];
      for (uint64_t j = 0; j < d; j++) S[i * d + j] = a * S[i * d + j] + ki * (double)v[t * d + j];
    }
    for (uint64_t j = 0; j < d; j++) {
      double acc = 0.0;
      for (uint64_t i = 0; i < d; i++) acc += (double)q[t * d + i] * S[i * d + j];
      out[t * d + j] = scale * acc;
    }
  }
  free(S);
}

/* The same head computed the way the kernel is written (examples/kda_fp32.ph:27-64): chunks of
 * `c` tokens, b = cumsum(g), qd = q*exp(b)*scale, kd = k*exp(-b), P = tril(qd kd^T),
 * o = P v + qd S, S = S*exp(total) + (k*exp(total - b))^T v, in f64. */
PH_EXPORT void ph_oracle_kda_chunked(const float *q, const float *k, const float *v, const float *g, uint64_t n, uint64_t d,
                                    uint64_t c, double scale, double *out) {
  double *S = (double *)calloc(d * d, sizeof(double));
  double *b = (double *)malloc(c * sizeof(double));
  double *qd = (double *)malloc(c * d * sizeof(double));
  double *kd = (double *)malloc(c * d * sizeof(double));
  double *kf = (double *)malloc(c * d * sizeof(double));
  double *Sn = (double *)malloc(d * d * sizeof(double));
  for (uint64_t c0 = 0; c0 < n; c0 += c) {
    const uint64_t rows = n - c0 < c ? n - c0 : c;
    double run = 0.0;
    for (uint64_t r = 0; r < rows; r++) {
      run += (double)g[c0 + r];
      b[r] = run;
    }
    const double total = run;
    for (uint64_t r = 0; r < rows; r++)
      for (uint64_t x = 0; x < d; x++) {
        qd[r * d + x] = (double)q[(c0 + r) * d + x] * exp(b[r]) * scale;
        kd[r * d + x] = (double)k[(c0 + r) * d + x] * exp(-b[r]);
        kf[r * d + x] = (double)k[(c0 + r) * d + x] * exp(total - b[r]);
      }
    for (uint64_t i = 0; i < rows; i++)
      for (uint64_t x = 0; x < d; x++) {
        double acc = 0.0;
        for (uint64_t j = 0; j <= i; j++) {
          double pij = 0.0;
          for (uint64_t y = 0; y < d; y++) pij += qd[i * d + y] * kd[j * d + y];
          acc += pij * (double)v[(c0 + j) * d + x];
        }
        for (uint64_t y = 0; y < d; y++) acc += qd[i * d + y] * S[y * d + x];
        out[(c0 + i) * d + x] = acc;
      }
    for (uint64_t i = 0; i < d; i++)
      for (uint64_t x = 0; x < d; x++) {
        double acc = S[i * d + x] * exp(total);
        for (uint64_t j = 0; j < rows; j++) acc += kf[j * d + i] * (double)v[(c0 + j) * d + x];
        Sn[i * d + x] = acc;
      }
    memcpy(S, Sn, d * d * sizeof(double));
  }
  free(S); free(b); free(qd); free(kd); free(kf); free(Sn);
}

/* verify_saxpy (phobos-bench/src/main.rs:1179-1188): want[i] = alpha * x[i] + y[i] in f32, a
 * rounded product and then a rounded sum (the volatile keeps the compiler from fusing them). */
PH_EXPORT void ph_oracle_saxpy(const float *x, const float *y, float alpha, uint64_t n, float *out) {
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < n; i++) {
    volatile float prod = alpha * x[i];
    out[i] = prod + y[i];
  }
}

PH_EXPORT double ph_oracle_rel_frobenius(const float *got, const double *want, uint64_t n) {
  double num = 0.0, den = 0.0;
#pragma omp parallel for reduction(+ : num, den) schedule(static)
  for (uint64_t i = 0; i < n; i++) {
    double d = (double)got[i] - want[i];
    num += d * d;
    den += want[i] * want[i];
  }
  return den > 0.0 ? sqrt(num / den) : sqrt(num);
}

/* max over elements of |got-want| / max(|want|, floor): the reference's
 * sampled criterion (main.rs:438, 913; cluster_correctness.rs:97-125). */
PH_EXPORT double ph_oracle_max_rel_floor(const float *got, const double *want, uint64_t n, double floor_) {
  double worst = 0.0;
#pragma omp parallel for reduction(max : worst) schedule(static)
  for (uint64_t i = 0; i < n; i++) {
    double w = fabs(want[i]);
    double rel = fabs((double)got[i] - want[i]) / (w > floor_ ? w : floor_);
    if (rel > worst) worst = rel;
  }
  return worst;
}

PH_EXPORT int ph_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of threads of the following parallel regions (a launcher may have exported
 * OMP_NUM_THREADS=1 for its worker processes). */
PH_EXPORT void ph_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
