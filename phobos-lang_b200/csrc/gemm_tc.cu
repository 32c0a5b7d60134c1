// Tensor-core GEMM for sm_100a: C = alpha * A@B + beta * C with f16 A and B.
//
// Covers the reference's `gemm` kernel in its two tensor-core regimes
//   gemm_fp16tc_fp32acc  (examples/gemm_fp16tc_fp32acc.ph; f32 accumulate, f32 C;
//                         emit_mma_sync_matmul, phobos-lang/src/codegen/matmul.rs:1229-1276)
//   gemm_fp16            (examples/gemm_fp16.ph; f16 accumulate, f16 C, f32 epilogue;
//                         DrainMode::VecF16, matmul.rs:1015-1025)
// as one persistent, warp-specialised kernel:
//   warp 0      TMA producer: A tile [128 x 64] (K-major) and B tile [64 x BN]
//               (N-major, straight from the row-major B) into 128B-swizzled
//               shared-memory stages, one mbarrier per stage
//   warp 1      tcgen05.mma issuer (one thread), accumulators in tensor memory,
//               two accumulator buffers so the epilogue of tile i overlaps the
//               main loop of tile i+1
//   warps 2..5  epilogue: tcgen05.ld -> alpha*acc + beta*C_old -> global
// A is [M,K] row-major and B is [K,N] row-major, exactly the .ph layout; B is
// consumed as an MN-major UMMA operand, so no transpose pass exists.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 f16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BK * BN * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 8 ? 8 : (SMEM_BUDGET / STAGE_BYTES);
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct TcParams {
  int M, N, K;
  int tiles_m, tiles_n;
  float alpha, beta;
  void* C;
  long long ldc;
  uint32_t* status;
};

// Tiles are walked in bands of 8 row-blocks so that concurrently resident CTAs
// share A row-panels and B column-panels in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  constexpr int GROUP = 8;
  const int per_group = GROUP * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(GROUP, tiles_m - first_m);
  const int r = t - g * per_group;
  mb = first_m + r % gsize;
  nb = r / gsize;
}

template <int BN, bool ACC_F16, typename CT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, TcParams p) {
  using C_ = Cfg<BN>;
  constexpr int STAGES = C_::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // rounded up to 1024 B as an offset into the array: a pointer rebuilt from an integer would lose the
  // shared address space and turn every access through it into a generic load or store
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * C_::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C_::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wctx{abort_flag, p.status};
  __shared__ unsigned long long clock_slot[2];
  const bool clock_cta = threadIdx.x == 0 && blockIdx.x == 0;
  if (clock_cta) launch_clock_begin(clock_slot);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty[stage], phase ^ 1, SITE_GEMM_PRODUCER_EMPTY, wctx)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[stage], C_::STAGE_BYTES);
          tma_load_2d(sA + stage * C_::A_BYTES, &tmA, &full[stage], kb * BK, mb * BM);
#pragma unroll
          for (int j = 0; j < BN / 64; j++)
            tma_load_2d(sB + stage * C_::B_BYTES + j * (BK * 128), &tmB, &full[stage], nb * BN + j * 64, kb * BK);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, BN, !ACC_F16, /*a_mn=*/false, /*b_mn=*/true);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, SITE_GEMM_MMA_TMEM_EMPTY, wctx)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full[stage], phase, SITE_GEMM_MMA_FULL, wctx)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * C_::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * C_::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            // A: K-major, 128B swizzle: 8-row groups 1024 B apart; a K step of 16
            // elements is 32 B inside the swizzle row.
            const uint64_t a_desc = umma_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            // B: N-major, 128B swizzle: a row of 64 n-values per k; 8 k-rows form a
            // 1024 B atom (stride offset), 64-column groups are BK*128 B apart
            // (leading offset); a K step of 16 is two atoms = 2048 B.
            const uint64_t b_desc = umma_smem_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024);
            umma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      // the vote keeps the warp together: the TMEM loads below are warp-collective
      if (!PH_WARP_WAIT(&tmem_full[acc], acc_phase, SITE_GEMM_EPI_TMEM_FULL, wctx)) break;
      tc_fence_after_sync();
      const int row = mb * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      CT* crow = reinterpret_cast<CT*>(p.C) + static_cast<long long>(row) * p.ldc;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c * 32;
        if (row_ok && col0 < p.N) {
          if constexpr (sizeof(CT) == 4) {
#pragma unroll
            for (int v = 0; v < 8; v++) {
              const int col = col0 + v * 4;
              if (col < p.N) {  // N is a multiple of 4
                float4 old = *reinterpret_cast<const float4*>(crow + col);
                float4 o;
                o.x = __fadd_rn(__fmul_rn(p.alpha, __uint_as_float(r[v * 4 + 0])), __fmul_rn(p.beta, old.x));
                o.y = __fadd_rn(__fmul_rn(p.alpha, __uint_as_float(r[v * 4 + 1])), __fmul_rn(p.beta, old.y));
                o.z = __fadd_rn(__fmul_rn(p.alpha, __uint_as_float(r[v * 4 + 2])), __fmul_rn(p.beta, old.z));
                o.w = __fadd_rn(__fmul_rn(p.alpha, __uint_as_float(r[v * 4 + 3])), __fmul_rn(p.beta, old.w));
                *reinterpret_cast<float4*>(crow + col) = o;
              }
            }
          } else {
#pragma unroll
            for (int v = 0; v < 4; v++) {
              const int col = col0 + v * 8;
              if (col < p.N) {  // N is a multiple of 8
                uint4 oldv = *reinterpret_cast<const uint4*>(crow + col);
                const __half2* oh = reinterpret_cast<const __half2*>(&oldv);
                uint4 outv;
                __half2* outh = reinterpret_cast<__half2*>(&outv);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                  float a0, a1;
                  if constexpr (ACC_F16) {
                    a0 = __half2float(__ushort_as_half(static_cast<unsigned short>(r[v * 8 + 2 * e] & 0xFFFF)));
                    a1 = __half2float(__ushort_as_half(static_cast<unsigned short>(r[v * 8 + 2 * e + 1] & 0xFFFF)));
                  } else {
                    a0 = __uint_as_float(r[v * 8 + 2 * e]);
                    a1 = __uint_as_float(r[v * 8 + 2 * e + 1]);
                  }
                  const float2 of = __half22float2(oh[e]);
                  const float x = __fadd_rn(__fmul_rn(p.alpha, a0), __fmul_rn(p.beta, of.x));
                  const float y = __fadd_rn(__fmul_rn(p.alpha, a1), __fmul_rn(p.beta, of.y));
                  outh[e] = __floats2half2_rn(x, y);
                }
                *reinterpret_cast<uint4*>(crow + col) = outv;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------ teardown --------------------------------------
  __syncwarp();
  if (*abort_flag != 0) {
    // a wait gave up: give copies and MMAs still in flight time to land before
    // shared and tensor memory are released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, C_::TMEM_COLS);
  if (clock_cta) launch_clock_end(clock_slot, p.status);
}

}  // namespace

template <int BN, bool ACC_F16, typename CT>
static cudaError_t launch_cfg(const CUtensorMap& tmA, const CUtensorMap& tmB, TcParams p, int sm_count,
                              cudaStream_t stream) {
  using C_ = Cfg<BN>;
  auto kern = gemm_tc_kernel<BN, ACC_F16, CT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, NUM_THREADS, C_::SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError();
}

// A: [M,K] f16 row-major (lda), B: [K,N] f16 row-major (ldb), C: [M,N] f32 or f16 (ldc).
int launch_gemm_tc(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                   int K, float alpha, float beta, bool acc_f16, bool c_f16, int sm_count,
                   uint32_t* status, cudaStream_t stream, const char** err) {
  CUtensorMap tmA, tmB;
  if (!make_tmap_2d(&tmA, A, TMAP_F16, M, K, lda, BM, BK, TMAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tmB, B, TMAP_F16, K, N, ldb, BK, 64, TMAP_SWIZZLE_128B)) {
    *err = "cuTensorMapEncodeTiled failed (alignment or driver entry point)";
    return -1;
  }
  TcParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.alpha = alpha;
  p.beta = beta;
  p.C = C;
  p.ldc = ldc;
  p.status = status;
  int bn;
  {
    // widest tile that still fills the machine in whole waves reasonably well
    auto waste = [&](int b) {
      long long tiles = static_cast<long long>((M + BM - 1) / BM) * ((N + b - 1) / b);
      long long waves = (tiles + sm_count - 1) / sm_count;
      return static_cast<double>(tiles) / static_cast<double>(waves * sm_count);
    };
    bn = 256;
    if (N <= 64) bn = 64;
    else if (N <= 128) bn = 128;
    else if (waste(256) < 0.9 && waste(128) > waste(256) + 0.05) bn = 128;
  }
  cudaError_t e;
  if (!acc_f16 && !c_f16) {
    e = bn == 256 ? launch_cfg<256, false, float>(tmA, tmB, p, sm_count, stream)
        : bn == 128 ? launch_cfg<128, false, float>(tmA, tmB, p, sm_count, stream)
                    : launch_cfg<64, false, float>(tmA, tmB, p, sm_count, stream);
  } else if (acc_f16 && c_f16) {
    e = bn == 256 ? launch_cfg<256, true, __half>(tmA, tmB, p, sm_count, stream)
        : bn == 128 ? launch_cfg<128, true, __half>(tmA, tmB, p, sm_count, stream)
                    : launch_cfg<64, true, __half>(tmA, tmB, p, sm_count, stream);
  } else {
    *err = "unsupported accumulator / output type combination";
    return -2;
  }
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
