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
// Structure: CTA tile 128x128, K step 16, 128 threads, 8 rows x 16 columns of outputs per
// thread in registers (128 accumulators as 64 packed pairs), two CTAs per SM.  A [128 x 16]
// and B [16 x 128] tiles are staged by TMA into a ring of shared-memory stages; a `full`
// mbarrier per stage signals arrival and an `empty` mbarrier (one arrival per warp) lets the
// refill proceed without a CTA-wide barrier, so warps drift apart by up to a stage.  The A
// tile is stored 64B-swizzled so that the rows a warp reads in one instruction land in
// different banks.  The multiply-adds are issued as packed fma.rn.f32x2 (two independent
// IEEE fmas per instruction): the math is unchanged while the instruction count halves.
//
// Why 8 x 16 per thread: a shared-memory wavefront delivers 4 bytes per lane, so a thread
// tile of r x c outputs needs r + c wavefronts per k for r * c fmas.  The SM does 128 fmas
// and 1 wavefront per clock, i.e. 4 fmas per lane per wavefront at balance: an 8 x 8 tile
// sits exactly on that line (measured: 540 M shared wavefronts, the load pipe as busy as
// the FMA pipe, 48 TFLOP/s), 8 x 16 needs 24 wavefronts per 128 fmas (75 %; 52 TFLOP/s).
// The price is 255 registers per thread, hence two warps per scheduler.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int STAGES = 4;
constexpr int THREADS = 128;
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

// acc (+)= a * b on both 32-bit halves: two fma.rn.f32 in one instruction.
__device__ __forceinline__ void ffma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long dup2(float x) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float2 unpack2(unsigned long long v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}

__global__ void __launch_bounds__(THREADS, 2)
gemm_f32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, F32Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(empty + STAGES);
  const WaitCtx wctx{abort_flag, p.status};
  // a CTA of the last quarter of the grid reports the SM clock it saw
  __shared__ unsigned long long clock_slot[2];
  const bool clock_cta = threadIdx.x == 0 && blockIdx.x == (gridDim.x - 1 - (gridDim.x >> 2));
  if (clock_cta) launch_clock_begin(clock_slot);

  // Tile of this CTA.  CTAs are dispatched in index order, about two per SM at a time, and the tiles in flight
  // walk K together, so an A or B k-slab fetched from DRAM by one of them is an L2 hit for the others that
  // share its row or column block.  DRAM traffic per "wave" is therefore (rows + columns of the block of tiles
  // in flight) panels: bands of 16 tile rows, odd bands walked right to left, make that block about square
  // (16 x 18 for 296 tiles in flight; bands of 8 read a third more).
  int mb, nb;
  {
    constexpr int GROUP = 16;
    const int t = blockIdx.x;
    const int per_group = GROUP * p.tiles_n;
    const int g = t / per_group;
    const int first_m = g * GROUP;
    const int gsize = min(GROUP, p.tiles_m - first_m);
    const int r = t - g * per_group;
    mb = first_m + r % gsize;
    nb = r / gsize;
    if (g & 1) nb = p.tiles_n - 1 - nb;
  }

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // warp tile 64 rows x 64 cols; warps arranged 2 (rows) x 2 (cols); 8 rows x 16 columns per thread
  const int wrow = (warp >> 1) * 64, wcol = (warp & 1) * 64;
  const int ty = lane >> 2;  // 0..7 : rows  wrow + ty + 8*i
  const int tx = lane & 3;   // 0..3 : cols  wcol + tx*4 + 16*j + (0..3)

  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], THREADS / 32);
    }
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

  // acc[i][jp]: row wrow + ty + 8*i, column pair jp (columns 2*jp, 2*jp+1 of the thread's 16)
  unsigned long long acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int jp = 0; jp < 8; jp++) acc[i][jp] = 0ull;  // two +0.0f

  // byte offset of row (wrow + ty + 4*i) in an A tile and its swizzle term:
  // row r lives at r*64 B, its 16-byte chunk c at chunk (c ^ ((r >> 1) & 3))  (TMA 64B swizzle)
  const int a_row_base = (wrow + ty) * 64;
  const int b_col_base = (wcol + tx * 4) * 4;

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int kb = 0; kb < num_kb; kb++) {
    // refill the stage consumed one iteration ago, once every warp has released it
    if (tid == 0 && kb >= 1 && kb - 1 + STAGES < num_kb) {
      const int ps = (stage + STAGES - 1) % STAGES;
      const uint32_t pphase = (ps == STAGES - 1) ? (phase ^ 1) : phase;  // phase of iteration kb-1
      if (mbar_wait(&empty[ps], pphase, SITE_GEMM_PRODUCER_EMPTY, wctx)) issue(kb - 1 + STAGES, ps);
    }
    if (!mbar_wait(&full[stage], phase, SITE_GEMM_MMA_FULL, wctx)) {
      ok = false;
      break;
    }
    const uint8_t* sA = smem + stage * STAGE_BYTES;
    const uint8_t* sB = smem + stage * STAGE_BYTES + A_BYTES;
#pragma unroll
    for (int k2 = 0; k2 < BK / 2; k2++) {
      // two k at a time: a 64-bit load per row (rows of a warp sit in different banks thanks to
      // the swizzle), four 128-bit loads of B per k
      const int kc = k2 >> 1, half = k2 & 1;
      float2 a[8];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int r = wrow + ty + 8 * i;
        a[i] = *reinterpret_cast<const float2*>(sA + a_row_base + i * 512 + ((kc ^ ((r >> 1) & 3)) << 4) + half * 8);
      }
#pragma unroll
      for (int kk = 0; kk < 2; kk++) {
        const uint8_t* brow = sB + (k2 * 2 + kk) * (BN * 4) + b_col_base;
        ulonglong2 b[4];
#pragma unroll
        for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const ulonglong2*>(brow + j * 64);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const unsigned long long a2 = dup2(kk == 0 ? a[i].x : a[i].y);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            ffma2(acc[i][2 * j], a2, b[j].x);
            ffma2(acc[i][2 * j + 1], a2, b[j].y);
          }
        }
      }
    }
    // this warp is done with the stage
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);
    if (++stage == STAGES) {
      stage = 0;
      phase ^= 1;
    }
  }

  if (ok) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = mb * BM + wrow + ty + 8 * i;
      if (row < p.M) {
        float* crow = p.C + static_cast<long long>(row) * p.ldc;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int col = nb * BN + wcol + tx * 4 + 16 * j;
          if (col < p.N) {  // N is a multiple of 4
            const float4 old = *reinterpret_cast<const float4*>(crow + col);
            const float2 lo = unpack2(acc[i][2 * j]), hi = unpack2(acc[i][2 * j + 1]);
            float4 o;
            o.x = __fadd_rn(__fmul_rn(p.alpha, lo.x), __fmul_rn(p.beta, old.x));
            o.y = __fadd_rn(__fmul_rn(p.alpha, lo.y), __fmul_rn(p.beta, old.y));
            o.z = __fadd_rn(__fmul_rn(p.alpha, hi.x), __fmul_rn(p.beta, old.z));
            o.w = __fadd_rn(__fmul_rn(p.alpha, hi.y), __fmul_rn(p.beta, old.w));
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
  if (clock_cta) launch_clock_end(clock_slot, p.status);
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
