// Chunkwise gated linear attention ("kda"), the reference's examples/kda_fp32.ph:1-65.
//
// One program streams one head's sequence in chunks of C tokens and carries the [D, D]
// state S across chunks.  With g the per-token log forget-gate and b its inclusive prefix
// sum inside the chunk (the `cumsum` builtin, SPEC.md, "Built-Ins"):
//   qd = q * exp(b) * scale          kd = k * exp(-b)
//   P  = tril(qd @ kd^T)             (keep j <= i; the `tril` builtin)
//   O[chunk] = P @ v + qd @ S
//   total = sum of the chunk's g     kfin = k * exp(total - b)
//   S  = S * exp(total) + kfin^T @ v (the `transpose` builtin feeds the contraction over tokens)
// All arithmetic is f32; exp is ex2.approx.ftz of x * log2(e), as the reference lowers
// `exp` (phobos-lang/src/codegen/tile.rs:1033-1061).  The kernel's signature has no batch or
// head axis and no program_id, so a launch is a single program, as in the reference: this
// is one CTA whose 256 threads share the chunk's tiles in shared memory.  It is a
// correctness leaf (the reference neither benchmarks nor verifies it numerically), not a
// tuned kernel.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int KD_D = 64;        // head dim (the kernel's `D in [64]`)
constexpr int KD_C = 64;        // tokens per chunk (a choice inside the kernel's `C in [32, 128]`)
constexpr int KD_THREADS = 256;

__device__ __forceinline__ float exp_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

struct KdaParams {
  const float* Q;
  const float* K;
  const float* V;
  const float* G;
  float* O;
  long long ldq, ldk, ldv, ldg, ldo;
  int N;
  float scale;
};

__global__ void __launch_bounds__(KD_THREADS, 1) kda_kernel(KdaParams p) {
  extern __shared__ float sm[];
  float* sQ = sm;                       // [C][D]   q, then qd
  float* sK = sQ + KD_C * KD_D;         // [C][D]   k, then kd
  float* sV = sK + KD_C * KD_D;         // [C][D]
  float* sF = sV + KD_C * KD_D;         // [C][D]   kfin
  float* sP = sF + KD_C * KD_D;         // [C][C+1] (padded: column reads)
  float* sS = sP + KD_C * (KD_C + 1);   // [D][D]   state
  float* sB = sS + KD_D * KD_D;         // [C]      inclusive prefix sums of g
  const int tid = threadIdx.x;

  for (int i = tid; i < KD_D * KD_D; i += KD_THREADS) sS[i] = 0.0f;
  __syncthreads();

  for (int c0 = 0; c0 < p.N; c0 += KD_C) {
    const int rows = min(KD_C, p.N - c0);   // tokens of this chunk that exist
    // ---- load the chunk (rows past the end read as zero, as masked slices do) -------------
    for (int i = tid; i < KD_C * KD_D; i += KD_THREADS) {
      const int r = i / KD_D, d = i - r * KD_D;
      const bool in = r < rows;
      sQ[i] = in ? p.Q[static_cast<long long>(c0 + r) * p.ldq + d] : 0.0f;
      sK[i] = in ? p.K[static_cast<long long>(c0 + r) * p.ldk + d] : 0.0f;
      sV[i] = in ? p.V[static_cast<long long>(c0 + r) * p.ldv + d] : 0.0f;
    }
    if (tid < KD_C) sB[tid] = tid < rows ? p.G[static_cast<long long>(c0 + tid) * p.ldg] : 0.0f;
    __syncthreads();
    // ---- cumsum down the chunk (inclusive), by one thread in token order --------------------
    if (tid == 0) {
      float run = 0.0f;
      for (int r = 0; r < KD_C; r++) {
        run = __fadd_rn(run, sB[r]);
        sB[r] = run;
      }
    }
    __syncthreads();
    const float total = sB[KD_C - 1];
    // ---- decay-folded queries and keys -----------------------------------------------------------
    for (int i = tid; i < KD_C * KD_D; i += KD_THREADS) {
      const int r = i / KD_D;
      const float b = sB[r];
      const float k = sK[i];
      sQ[i] = sQ[i] * exp_approx(b) * p.scale;
      sK[i] = k * exp_approx(-b);
      sF[i] = k * exp_approx(total - b);
    }
    __syncthreads();
    // ---- P = tril(qd @ kd^T): thread (ti, tj) computes a 4 x 4 block -----------------------------
    {
      const int ti = (tid >> 4) * 4, tj = (tid & 15) * 4;
      float acc[4][4] = {};
      if (tj <= ti + 3) {   // blocks strictly above the diagonal stay zero
        for (int d = 0; d < KD_D; d++) {
          float a[4], b[4];
#pragma unroll
          for (int x = 0; x < 4; x++) {
            a[x] = sQ[(ti + x) * KD_D + d];
            b[x] = sK[(tj + x) * KD_D + d];
          }
#pragma unroll
          for (int x = 0; x < 4; x++)
#pragma unroll
            for (int y = 0; y < 4; y++) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
        }
      }
#pragma unroll
      for (int x = 0; x < 4; x++)
#pragma unroll
        for (int y = 0; y < 4; y++) sP[(ti + x) * (KD_C + 1) + tj + y] = (tj + y <= ti + x) ? acc[x][y] : 0.0f;
    }
    __syncthreads();
    // ---- O = P @ v + qd @ S: thread computes a 4 x 4 block of [C][D] ----------------------------------
    {
      const int ti = (tid >> 4) * 4, tj = (tid & 15) * 4;
      float acc[4][4] = {};
      for (int j = 0; j < KD_C; j++) {
        float a[4], b[4];
#pragma unroll
        for (int x = 0; x < 4; x++) {
          a[x] = sP[(ti + x) * (KD_C + 1) + j];
          b[x] = sV[j * KD_D + tj + x];
        }
#pragma unroll
        for (int x = 0; x < 4; x++)
#pragma unroll
          for (int y = 0; y < 4; y++) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
      }
      for (int d = 0; d < KD_D; d++) {
        float a[4], b[4];
#pragma unroll
        for (int x = 0; x < 4; x++) {
          a[x] = sQ[(ti + x) * KD_D + d];
          b[x] = sS[d * KD_D + tj + x];
        }
#pragma unroll
        for (int x = 0; x < 4; x++)
#pragma unroll
          for (int y = 0; y < 4; y++) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
      }
#pragma unroll
      for (int x = 0; x < 4; x++)
        if (ti + x < rows) {
          float4 o = make_float4(acc[x][0], acc[x][1], acc[x][2], acc[x][3]);
          *reinterpret_cast<float4*>(p.O + static_cast<long long>(c0 + ti + x) * p.ldo + tj) = o;
        }
    }
    __syncthreads();   // every read of the old state is done
    // ---- S = S * exp(total) + kfin^T @ v: thread computes a 4 x 4 block of [D][D] ---------------------
    {
      const int ti = (tid >> 4) * 4, tj = (tid & 15) * 4;
      const float decay = exp_approx(total);
      float acc[4][4];
#pragma unroll
      for (int x = 0; x < 4; x++)
#pragma unroll
        for (int y = 0; y < 4; y++) acc[x][y] = 0.0f;
      for (int j = 0; j < KD_C; j++) {
        float a[4], b[4];
#pragma unroll
        for (int x = 0; x < 4; x++) {
          a[x] = sF[j * KD_D + ti + x];
          b[x] = sV[j * KD_D + tj + x];
        }
#pragma unroll
        for (int x = 0; x < 4; x++)
#pragma unroll
          for (int y = 0; y < 4; y++) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
      }
#pragma unroll
      for (int x = 0; x < 4; x++)
#pragma unroll
        for (int y = 0; y < 4; y++) {
          float* s = &sS[(ti + x) * KD_D + tj + y];
          *s = __fadd_rn(__fmul_rn(*s, decay), acc[x][y]);
        }
    }
    __syncthreads();
  }
}

}  // namespace

int launch_kda(const float* Q, long long ldq, const float* K, long long ldk, const float* V, long long ldv, const float* G,
               long long ldg, float* O, long long ldo, int N, int D, float scale, cudaStream_t stream, const char** err) {
  if (D != KD_D) {
    *err = "kda: head dim must be 64";
    return -2;
  }
  KdaParams p{Q, K, V, G, O, ldq, ldk, ldv, ldg, ldo, N, scale};
  const size_t smem = (4 * KD_C * KD_D + KD_C * (KD_C + 1) + KD_D * KD_D + KD_C) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(kda_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e == cudaSuccess) {
    kda_kernel<<<1, KD_THREADS, smem, stream>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
