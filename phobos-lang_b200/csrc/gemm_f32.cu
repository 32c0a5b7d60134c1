// FP32 GEMM on the CUDA cores (FFMA, no TF32) and the matmul_init leaf.
//
// Covers the reference's `gemm` f32 kernel (examples/gemm_fp32.ph:1-22;
// emit_register_matmul, phobos-lang/src/codegen/matmul.rs:639-741) and the
// partitioned `matmul` step leaf (examples/matmul_cluster_fp32.ph:1-17), whose
// arithmetic is: accumulator 0, one fma.rn per multiply-add with k ascending,
// then alpha*acc + beta*C_old as mul, mul, add in f32 (matmul.rs:384-403,
// phobos-lang/src/codegen/tile.rs:1790-1794).  This kernel keeps that exact
// per-element operation order, so on the same inputs the result is bit-identical
// to a sequential f32 fma chain.
//
// Structure: CTA tile 128x128, K step 16, 256 threads, 8x8 outputs per thread in
// registers.  A [128 x 16] and B [16 x 128] tiles are staged by TMA into a
// 4-deep ring of shared-memory stages (one elected thread issues, mbarriers
// signal arrival); fragments are read with 128-bit shared loads.  The A tile is
// stored 64B-swizzled so that the four rows a warp reads in one instruction land
// in different banks.  Two CTAs are resident per SM.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int STAGES = 4;
constexpr int THREADS = 256;
constexpr int A_BYTES = BM * BK * 4;  // 8 KB
constexpr int B_BYTES = BK * BN * 4;  // 8 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 128;

struct F32Params {
  int M, N, K;
  int tiles_m, tiles_n;
  float alpha, beta;
  float* C;
  long long ldc;
  uint32_t* status;
};

__global__ void __launch_bounds__(THREADS, 2)
gemm_f32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, F32Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(full + STAGES);
  const WaitCtx wctx{abort_flag, p.status};

  // tile of this CTA: bands of 8 row-blocks for L2 reuse
  int mb, nb;
  {
    constexpr int GROUP = 8;
    const int t = blockIdx.x;
    const int per_group = GROUP * p.tiles_n;
    const int g = t / per_group;
    const int first_m = g * GROUP;
    const int gsize = min(GROUP, p.tiles_m - first_m);
    const int r = t - g * per_group;
    mb = first_m + r % gsize;
    nb = r / gsize;
  }

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // warp tile 32 rows x 64 cols; warps arranged 4 (rows) x 2 (cols)
  const int wrow = (warp >> 1) * 32, wcol = (warp & 1) * 64;
  const int ty = lane >> 3;  // 0..3 : rows  wrow + ty + 4*i
  const int tx = lane & 7;   // 0..7 : cols  wcol + tx*4 + 32*j + (0..3)

  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) mbar_init(&full[s], 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  __syncthreads();

  const int num_kb = (p.K + BK - 1) / BK;
  auto issue = [&](int kb, int stage) {
    mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
    tma_load_2d(smem + stage * STAGE_BYTES, &tmA, &full[stage], kb * BK, mb * BM);
    tma_load_2d(smem + stage * STAGE_BYTES + A_BYTES, &tmB, &full[stage], nb * BN, kb * BK);
  };
  if (tid == 0) {
    for (int s = 0; s < STAGES && s < num_kb; s++) issue(s, s);
  }

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

  // Per-row swizzled offsets inside an A tile: row r lives at r*64 B and its
  // 16-byte chunk c sits at chunk (c ^ ((r >> 1) & 3))  (TMA 64B swizzle).
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int kb = 0; kb < num_kb; kb++) {
    ok = mbar_wait(&full[stage], phase, SITE_GEMM_MMA_FULL, wctx);
    const uint8_t* sA = smem + stage * STAGE_BYTES;
    const float* sB = reinterpret_cast<const float*>(smem + stage * STAGE_BYTES + A_BYTES);
    if (ok) {
#pragma unroll
    for (int kc = 0; kc < BK / 4; kc++) {
      float4 a[8];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int r = wrow + ty + 4 * i;
        a[i] = *reinterpret_cast<const float4*>(sA + r * 64 + ((kc ^ ((r >> 1) & 3)) << 4));
      }
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        const float* brow = sB + (kc * 4 + kk) * BN + wcol + tx * 4;
        const float4 b0 = *reinterpret_cast<const float4*>(brow);
        const float4 b1 = *reinterpret_cast<const float4*>(brow + 32);
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float av = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
#pragma unroll
          for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av, b[j], acc[i][j]);
        }
      }
    }
    }
    // every thread is done reading this stage; the vote keeps the exit uniform
    // when a wait gave up
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) break;
    if (tid == 0 && kb + STAGES < num_kb) issue(kb + STAGES, stage);
    if (++stage == STAGES) {
      stage = 0;
      phase ^= 1;
    }
  }

  if (ok) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = mb * BM + wrow + ty + 4 * i;
      if (row < p.M) {
        float* crow = p.C + static_cast<long long>(row) * p.ldc;
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int col = nb * BN + wcol + tx * 4 + 32 * j;
          if (col < p.N) {  // N is a multiple of 4
            const float4 old = *reinterpret_cast<const float4*>(crow + col);
            float4 o;
            o.x = __fadd_rn(__fmul_rn(p.alpha, acc[i][4 * j + 0]), __fmul_rn(p.beta, old.x));
            o.y = __fadd_rn(__fmul_rn(p.alpha, acc[i][4 * j + 1]), __fmul_rn(p.beta, old.y));
            o.z = __fadd_rn(__fmul_rn(p.alpha, acc[i][4 * j + 2]), __fmul_rn(p.beta, old.z));
            o.w = __fadd_rn(__fmul_rn(p.alpha, acc[i][4 * j + 3]), __fmul_rn(p.beta, old.w));
            *reinterpret_cast<float4*>(crow + col) = o;
          }
        }
      }
    }
  } else {
    // a wait gave up: let copies still in flight land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

// C = beta * C, or C = 0 (matmul_init leaf).  One float4 per thread per step.
__global__ void scale_f32_kernel(float* C, long long ldc, long long rows, long long cols4, float beta,
                                 int zero_fill) {
  const long long total = rows * cols4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols4, c = i - r * cols4;
    float4* ptr = reinterpret_cast<float4*>(C + r * ldc) + c;
    float4 v;
    if (zero_fill) {
      v = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      v = *ptr;
      v.x = __fmul_rn(beta, v.x);
      v.y = __fmul_rn(beta, v.y);
      v.z = __fmul_rn(beta, v.z);
      v.w = __fmul_rn(beta, v.w);
    }
    *ptr = v;
  }
}

}  // namespace

int launch_gemm_f32(const float* A, long long lda, const float* B, long long ldb, float* C, long long ldc, int M,
                    int N, int K, float alpha, float beta, uint32_t* status, cudaStream_t stream, const char** err) {
  CUtensorMap tmA, tmB;
  if (!make_tmap_2d(&tmA, A, TMAP_F32, M, K, lda, BM, BK, TMAP_SWIZZLE_64B) ||
      !make_tmap_2d(&tmB, B, TMAP_F32, K, N, ldb, BK, BN, TMAP_SWIZZLE_NONE)) {
    *err = "cuTensorMapEncodeTiled failed (alignment or driver entry point)";
    return -1;
  }
  F32Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.alpha = alpha;
  p.beta = beta;
  p.C = C;
  p.ldc = ldc;
  p.status = status;
  cudaError_t e = cudaFuncSetAttribute(gemm_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e == cudaSuccess) {
    gemm_f32_kernel<<<p.tiles_m * p.tiles_n, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

int launch_scale_f32(float* C, long long ldc, long long rows, long long cols, float beta, bool zero_fill,
                     cudaStream_t stream, const char** err) {
  const long long cols4 = cols / 4;
  const long long total = rows * cols4;
  if (total == 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  scale_f32_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(C, ldc, rows, cols4, beta, zero_fill ? 1 : 0);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
