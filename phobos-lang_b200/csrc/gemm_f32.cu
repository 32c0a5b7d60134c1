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
// thread in registers (128 accumulators as 64 packed pairs), two or three CTAs per SM.  A and B tiles
// of 16 k are staged by TMA into a ring of shared-memory stages; a `full` mbarrier per stage
// signals arrival and an `empty` mbarrier (one arrival per warp) lets the refill proceed
// without a CTA-wide barrier, so warps drift apart by up to a stage.  The multiply-adds are
// issued as packed fma.rn.f32x2 (two independent IEEE fmas per instruction): the math is
// unchanged while the instruction count halves.
//
// Two forms of the same kernel, bit-identical results:
//  * AT (the caller gave workspace): a pass first writes A transposed, [K][M], into the
//    workspace, and the A tile lands in shared memory as [k][m].  A thread then fetches its
//    eight rows of one k with two 128-bit loads, as it fetches its sixteen columns of B with
//    four, and 24 fragment registers per k leave the compiler room to run the loads well ahead
//    of the multiply-adds.  The inner loop alone (shared memory preloaded, no barriers) runs at
//    67 TFLOP/s on a B200, 0.90 of the FFMA peak.
//  * in place (no workspace): the A tile is [m][k] as it lies in memory, 64B-swizzled so that
//    the rows a warp reads land in different banks; eight scalar loads per k (the inner loop
//    alone reaches 59-60 TFLOP/s in this layout whether the loads are scalar or 128-bit over
//    four k, which then hold 32 registers).
//
// Why 8 x 16 per thread: a shared-memory wavefront delivers 4 bytes per lane, so a thread
// tile of r x c outputs needs r + c wavefronts per k for r * c fmas.  The SM does 128 fmas
// and 1 wavefront per clock, i.e. 4 fmas per lane per wavefront at balance: an 8 x 8 tile
// sits exactly on that line, 8 x 16 needs 24 wavefronts per 128 fmas (75 %).
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

// AT: the A operand is the transposed copy [K][M] and its tile lands as [k][m].
// (the [k][m] form fits three CTAs per SM at 168 registers: +1 %)
template <bool AT>
__global__ void __launch_bounds__(THREADS, AT ? 3 : 2)
gemm_f32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, F32Params p) {
  extern __shared__ uint8_t smem_raw[];
  // rounded up to 1024 B as an offset into the array, so that the compiler still knows the address space
  // (a pointer rebuilt from an integer turns every fragment load into a generic load)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
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
  // in flight) panels: bands of 16 tile rows, odd bands walked right to left, keep that block compact
  // (16 x 18 for 296 tiles in flight, 16 x 28 for 444; bands of 8 read a third more).
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
  // In place: warp tile 64 x 64, warps 2 x 2; a thread has rows wrow + ty + 8*i and columns
  // wcol + 4*tx + 16*j + (0..3).
  // AT: a thread has rows 4*ty + (0..3) and 64 + 4*ty + (0..3), columns 4*tx + 32*j + (0..3), with
  // tx = tid % 8 and ty = tid / 8: both fragments of a k are 128-bit loads, and a warp stores whole
  // 128-byte row segments of C.
  const int wrow = AT ? 0 : (warp >> 1) * 64, wcol = AT ? 0 : (warp & 1) * 64;
  const int ty = AT ? (tid >> 3) : (lane >> 2);
  const int tx = AT ? (tid & 7) : (lane & 3);

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
    if constexpr (AT) tma_load_2d(smem + stage * STAGE_BYTES, &tmA, &full[stage], mb * BM, kb * BK);
    else tma_load_2d(smem + stage * STAGE_BYTES, &tmA, &full[stage], kb * BK, mb * BM);
    tma_load_2d(smem + stage * STAGE_BYTES + A_BYTES, &tmB, &full[stage], nb * BN, kb * BK);
  };
  if (tid == 0) {
    for (int s = 0; s < STAGES && s < num_kb; s++) issue(s, s);
  }

  // acc[i][jp]: i-th row of the thread, column pair jp (columns 2*jp, 2*jp+1 of the thread's 16)
  unsigned long long acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int jp = 0; jp < 8; jp++) acc[i][jp] = 0ull;  // two +0.0f

  // In place: byte offset of the thread's first row in an A tile; row r lives at r*64 B, its 16-byte chunk c
  // at chunk (c ^ ((r >> 1) & 3)) (TMA 64B swizzle), and that term is the same for the thread's eight rows.
  const int a_row_base = AT ? ty * 16 : (wrow + ty) * 64;
  const int b_col_base = AT ? tx * 16 : (wcol + tx * 4) * 4;
  uint32_t a_sw[4];
#pragma unroll
  for (int kc = 0; kc < 4; kc++) a_sw[kc] = static_cast<uint32_t>((kc ^ (((wrow + ty) >> 1) & 3)) << 4);

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
    if constexpr (AT) {
#pragma unroll
      for (int k = 0; k < BK; k++) {
        const float4 a0 = *reinterpret_cast<const float4*>(sA + k * (BM * 4) + a_row_base);
        const float4 a1 = *reinterpret_cast<const float4*>(sA + k * (BM * 4) + a_row_base + 256);
        ulonglong2 b[4];
#pragma unroll
        for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const ulonglong2*>(sB + k * (BN * 4) + b_col_base + j * 128);
        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const unsigned long long a2 = dup2(av[i]);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            ffma2(acc[i][2 * j], a2, b[j].x);
            ffma2(acc[i][2 * j + 1], a2, b[j].y);
          }
        }
      }
    } else {
      // one k at a time: eight scalar loads of A (the four lanes of a row share the word) and four 128-bit
      // loads of B; the fragments of k+1 are fetched before the multiply-adds of k are issued
      const uint32_t sA32 = smem_u32(sA) + a_row_base;
      const uint32_t sB32 = smem_u32(sB) + b_col_base;
      float a_cur[8], a_nxt[8];
      ulonglong2 b_cur[4], b_nxt[4];
      auto load_frag = [&](int k, float (&a)[8], ulonglong2 (&b)[4]) {
        const uint32_t aoff = a_sw[k >> 2] + (k & 3) * 4;
#pragma unroll
        for (int i = 0; i < 8; i++)
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a[i]) : "r"(sA32 + aoff + i * 512));
#pragma unroll
        for (int j = 0; j < 4; j++)
          asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];"
                       : "=l"(b[j].x), "=l"(b[j].y)
                       : "r"(sB32 + k * (BN * 4) + j * 64));
      };
      load_frag(0, a_cur, b_cur);
#pragma unroll
      for (int k = 0; k < BK; k++) {
        if (k + 1 < BK) load_frag(k + 1, a_nxt, b_nxt);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const unsigned long long a2 = dup2(a_cur[i]);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            ffma2(acc[i][2 * j], a2, b_cur[j].x);
            ffma2(acc[i][2 * j + 1], a2, b_cur[j].y);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) a_cur[i] = a_nxt[i];
#pragma unroll
        for (int j = 0; j < 4; j++) b_cur[j] = b_nxt[j];
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
      const int row = mb * BM + (AT ? 4 * ty + (i & 3) + 64 * (i >> 2) : wrow + ty + 8 * i);
      if (row < p.M) {
        float* crow = p.C + static_cast<long long>(row) * p.ldc;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int col = nb * BN + (AT ? 4 * tx + 32 * j : wcol + tx * 4 + 16 * j);
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

// At[k][m] = A[m][k]: 32 x 32 tiles through shared memory, both sides coalesced.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float* __restrict__ A, long long lda,
                                                            float* __restrict__ At, long long ldt, int M, int K) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int m = m0 + r, k = k0 + tx;
    tile[r][tx] = (m < M && k < K) ? A[static_cast<long long>(m) * lda + k] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int k = k0 + r, m = m0 + tx;
    if (k < K && m < M) At[static_cast<long long>(k) * ldt + m] = tile[tx][r];
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

size_t gemm_f32_workspace_bytes(long long M, long long K) {
  const long long ldt = (M + 3) / 4 * 4;
  return (static_cast<size_t>(K) * ldt * 4 + 255) & ~static_cast<size_t>(255);
}

int launch_gemm_f32(const float* A, long long lda, const float* B, long long ldb, float* C, long long ldc, int M,
                    int N, int K, float alpha, float beta, void* workspace, size_t workspace_bytes, uint32_t* status,
                    cudaStream_t stream, const char** err) {
  // with room for a transposed copy of A the A tile is read as [k][m]
  const bool at = workspace != nullptr && workspace_bytes >= gemm_f32_workspace_bytes(M, K) &&
                  reinterpret_cast<uintptr_t>(workspace) % 256 == 0;
  const long long ldt = (static_cast<long long>(M) + 3) / 4 * 4;
  CUtensorMap tmA, tmB;
  const bool maps = at ? make_tmap_2d(&tmA, workspace, TMAP_F32, K, M, ldt, BK, BM, TMAP_SWIZZLE_NONE)
                       : make_tmap_2d(&tmA, A, TMAP_F32, M, K, lda, BM, BK, TMAP_SWIZZLE_64B);
  if (!maps || !make_tmap_2d(&tmB, B, TMAP_F32, K, N, ldb, BK, BN, TMAP_SWIZZLE_NONE)) {
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
  cudaError_t e;
  if (at) {
    dim3 tgrid((K + 31) / 32, (M + 31) / 32);
    transpose_f32_kernel<<<tgrid, 256, 0, stream>>>(A, lda, static_cast<float*>(workspace), ldt, M, K);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_f32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) {
      gemm_f32_kernel<true><<<p.tiles_m * p.tiles_n, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
      e = cudaGetLastError();
    }
  } else {
    e = cudaFuncSetAttribute(gemm_f32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) {
      gemm_f32_kernel<false><<<p.tiles_m * p.tiles_n, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
      e = cudaGetLastError();
    }
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
