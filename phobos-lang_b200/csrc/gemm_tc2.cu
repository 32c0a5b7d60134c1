// Tensor-core GEMM for sm_100a on CTA pairs (tcgen05 cta_group::2):
// C = alpha * A@B + beta * C with f16 A and B.
//
// Same operator as gemm_tc.cu (the reference's `gemm` in its two tensor-core
// regimes, examples/gemm_fp16tc_fp32acc.ph and examples/gemm_fp16.ph), used for
// problems large enough to fill the machine.  Two CTAs on neighbouring SMs own
// one 256 x BN output tile: each CTA stages its own 128 rows of A and its own
// half of the B columns, so a CTA moves (128 + BN/2) * 64 operand elements per
// k-block into shared memory instead of (128 + BN) * 64 — the 1-CTA kernel is
// bound by that L2 -> shared-memory traffic, not by the tensor pipe.  One thread
// of the leader CTA issues the MMAs for the pair; completions are multicast to
// the mbarriers of both CTAs.  No TMA multicast is used: every CTA loads its
// own operand slices.
//
// Warp roles per CTA (256 threads): warp 0 TMA producer, warp 1 MMA issuer
// (leader CTA only) and tensor-memory owner, warps 2 and 3 the same two roles for
// an optional second tile in flight (idle by default), warps 4..7 epilogue
// (tcgen05.ld -> alpha*acc + beta*C_old -> global).  Two accumulator buffers of
// 256 columns let the epilogue of tile i overlap the main loop of tile i+1.
// BN is a run-time multiple of 16 (<= 256): 256 unless N is narrower.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int BM = 128;       // rows per CTA; 256 per pair
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 256;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_BYTES = BK * 128 * 2;         // 16 KB: up to 128 columns (two 64-column boxes) per CTA
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_LD = 36;                    // floats per row of an epilogue transpose pad (32 + 4: conflict-free)
constexpr int EPI_BYTES = 4 * 32 * EPI_LD * 4; // one 32 x 32 pad per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256;               // tensor-memory columns per accumulator buffer

struct Tc2Params {
  int M, N, K;
  int bn;                 // N extent of a pair tile
  int tiles_m, tiles_n;   // pair tiles
  int group_m;            // row-blocks per raster band
  float alpha, beta;
  void* C;
  long long ldc;
  uint32_t* status;
  // split-K of the last, partly filled round of tiles (f32 C only): the `split_tiles`
  // last tiles are each cut into `split` K ranges so that every CTA pair has work
  int split;            // 1 = off
  int split_first;      // index of the first split tile
  uint32_t* flags;      // hand-over words between the K ranges of a tile
  uint32_t epoch;       // distinguishes this launch's hand-overs from older ones
  // split-N of the last, partly filled round: its tiles are cut into two column halves (bn / 2 wide), so
  // that twice as many CTA pairs finish the launch together.  Unlike split-K the halves are independent.
  int nsplit;           // 1 = off, 2 = on (needs bn == 256; never together with split > 1)
  // 2: two tiles of a pair are in flight at once, each with its own producer, issuer,
  // accumulator buffer and half of the stage ring (see the kernel comment); 1: one tile
  int streams;
  int l2hint;             // bit 0: A panels loaded evict-last; bit 1: B panels evict-first; bit 2: C_old / C streaming
};

// Work unit u of a launch -> (tile, K range).  Units [0, split_first) are whole
// tiles; after them come `split` consecutive units per remaining tile.
struct Unit {
  int tile, part, kb0, kb1;
  int bn;        // width of this unit's output tile
  int col_off;   // its first column inside the tile's bn-wide column block
};
__device__ __forceinline__ Unit unit_of(int u, const Tc2Params& p, int num_kb) {
  Unit w;
  w.bn = p.bn;
  w.col_off = 0;
  if (u < p.split_first) {
    w.tile = u;
    w.part = 0;
    w.kb0 = 0;
    w.kb1 = num_kb;
  } else if (p.nsplit > 1) {
    const int v = u - p.split_first;
    w.tile = p.split_first + v / p.nsplit;
    w.part = v % p.nsplit;
    w.kb0 = 0;
    w.kb1 = num_kb;
    w.bn = p.bn / p.nsplit;
    w.col_off = w.part * w.bn;
  } else {
    const int v = u - p.split_first;
    w.tile = p.split_first + v / p.split;
    w.part = v % p.split;
    w.kb0 = static_cast<int>(static_cast<long long>(num_kb) * w.part / p.split);
    w.kb1 = static_cast<int>(static_cast<long long>(num_kb) * (w.part + 1) / p.split);
  }
  return w;
}
constexpr int FLAG_BANKS = 8, FLAG_TILES = 64;  // flags[bank][tile][cta][warp]
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int t, const Tc2Params& p, int& mb, int& nb) {
  const int per_group = p.group_m * p.tiles_n;
  const int g = t / per_group;
  const int first_m = g * p.group_m;
  const int gsize = min(p.group_m, p.tiles_m - first_m);
  const int r = t - g * per_group;
  mb = first_m + r % gsize;
  nb = r / gsize;
}

template <bool ACC_F16, typename CT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Tc2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                       // used in the leader CTA
  uint64_t* empty = bars + STAGES;             // one per CTA
  uint64_t* tmem_full = bars + 2 * STAGES;     // one per CTA
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // used in the leader CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* epi_pad = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();   // nothing above reads or writes global memory; everything below may

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_units = p.split_first + (num_tiles - p.split_first) * (p.nsplit > 1 ? p.nsplit : p.split);
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // Stream s (0 or 1) works on the pair's units n = s, s + streams, ... (unit n of a
  // pair is launch unit pair + n * num_pairs), accumulates into buffer n & 1 and owns
  // stages [s * ring, (s + 1) * ring) of the ring.
  const int ring = STAGES / p.streams;
  if (warp == 0 || warp == 2) {
    // ------------------------------ TMA producers (both CTAs) -------------------
    const int sidx = warp >> 1;
    if (lane == 0 && sidx < p.streams) {
      const int s0 = sidx * ring;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // a raster band's A rows are used by every wave of the band, a B panel by one wave only
      const uint64_t pol_a = l2_policy_evict_last(), pol_b = l2_policy_evict_first();
      for (int n = sidx; ok; n += p.streams) {
        const int u = pair + n * num_pairs;
        if (u >= num_units) break;
        const Unit w = unit_of(u, p, num_kb);
        int mb, nb;
        pair_tile_coords(w.tile, p, mb, nb);
        const int row0 = mb * (2 * BM) + static_cast<int>(rank) * BM;
        const int half_n = w.bn >> 1;                 // B columns staged by each CTA
        const int nbox = (half_n + 63) >> 6;
        const uint32_t stage_tx = 2u * static_cast<uint32_t>(A_BYTES + nbox * (BK * 128));
        const int col0 = nb * p.bn + w.col_off + static_cast<int>(rank) * half_n;
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          const int st = s0 + stage;
          if (!mbar_wait(&empty[st], phase ^ 1, SITE_GEMM_PRODUCER_EMPTY, wctx)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_u32(smem_u32(&full[st]), 0);
          if (leader) mbar_arrive_expect_tx(&full[st], stage_tx);  // bytes of both CTAs' loads
          if (p.l2hint & 1) tma_load_2d_pair_hint(sA + st * A_BYTES, &tmA, full_leader, kb * BK, row0, pol_a);
          else tma_load_2d_pair(sA + st * A_BYTES, &tmA, full_leader, kb * BK, row0);
          for (int j = 0; j < nbox; j++) {
            if (p.l2hint & 2)
              tma_load_2d_pair_hint(sB + st * B_BYTES + j * (BK * 128), &tmB, full_leader, col0 + j * 64, kb * BK, pol_b);
            else
              tma_load_2d_pair(sB + st * B_BYTES + j * (BK * 128), &tmB, full_leader, col0 + j * 64, kb * BK);
          }
          if (++stage == ring) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------ MMA issuers (leader CTA) ---------------------
    const int sidx = warp >> 1;
    if (leader && lane == 0 && sidx < p.streams) {
      const int s0 = sidx * ring;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int n = sidx; ok; n += p.streams) {
        const int u = pair + n * num_pairs;
        if (u >= num_units) break;
        const Unit w = unit_of(u, p, num_kb);
        const uint32_t idesc = umma_idesc_f16(2 * BM, w.bn, !ACC_F16, /*a_mn=*/false, /*b_mn=*/true);
        const int acc = n & 1;
        const uint32_t acc_phase = (n >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, SITE_GEMM_MMA_TMEM_EMPTY, wctx)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          const int st = s0 + stage;
          if (!mbar_wait(&full[st], phase, SITE_GEMM_MMA_FULL, wctx)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + st * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + st * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            const uint64_t a_desc = umma_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = umma_smem_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024);
            umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb != w.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[st], 0x3);  // both CTAs may refill this stage
          if (++stage == ring) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 0x3);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue (both CTAs) ---------------------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = pair; u < num_units; u += num_pairs) {
      const Unit w = unit_of(u, p, num_kb);
      int mb, nb;
      pair_tile_coords(w.tile, p, mb, nb);
      if (!PH_WARP_WAIT(&tmem_full[acc], acc_phase, SITE_GEMM_EPI_TMEM_FULL, wctx)) break;
      tc_fence_after_sync();
      // K range `part` of a split tile adds onto what range part-1 left in C: wait
      // for the hand-over word of this warp's 32 rows (same CTA rank, same warp)
      float beta = p.beta;
      uint32_t* flag = nullptr;
      if (p.split > 1 && u >= p.split_first) {
        flag = p.flags + ((((p.epoch % FLAG_BANKS) * FLAG_TILES + (w.tile - p.split_first)) * 2 + rank) * 4 + q);
        if (w.part > 0) {
          beta = 1.0f;
          uint32_t okw = 1;
          if (lane == 0) {
            const uint32_t want = p.epoch * 8u + static_cast<uint32_t>(w.part);
            const uint64_t t0 = globaltimer_ns();
            while (ld_acquire_u32(flag) != want) {
              if (globaltimer_ns() - t0 > PH_WAIT_NS) {
                okw = 0;
                *abort_flag = SITE_GEMM_EPI_TMEM_FULL;
                atomicCAS(p.status, 0u, SITE_GEMM_EPI_TMEM_FULL | (blockIdx.x << 8));
                break;
              }
            }
          }
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) break;
        }
      }
      const int row = mb * (2 * BM) + static_cast<int>(rank) * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      CT* crow = reinterpret_cast<CT*>(p.C) + static_cast<long long>(row) * p.ldc;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * ACC_STRIDE;
      const int tile_col0 = nb * p.bn + w.col_off;
      const int col_end = min(p.N, tile_col0 + w.bn);
      const int chunks = (w.bn + 31) >> 5;
      if constexpr (sizeof(CT) == 4) {
        // f32 C.  The accumulator arrives one row per lane; going to global memory that
        // way makes every warp instruction touch 32 different rows (16 useful bytes per
        // 32-byte sector, poor DRAM locality: measured 17 us per tile).  Each 32x32 chunk
        // is therefore transposed through a per-warp shared-memory pad so that a warp
        // instruction covers 4 rows x 128 contiguous bytes; the C_old values of the
        // chunk are requested before the transpose so their latency overlaps it.
        float* pad = epi_pad + q * (32 * EPI_LD);
        const bool cs = (p.l2hint & 4) != 0;
        const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;
        const long long row_base = static_cast<long long>(mb) * (2 * BM) + static_cast<int>(rank) * BM + q * 32;
#pragma unroll 1
        for (int c = 0; c < chunks; c++) {
          const int col = tile_col0 + c * 32 + sub_col;
          const bool col_ok = col < col_end;
          float4 old[8];
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const long long rr = row_base + it * 4 + sub_row;
            const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.C) + rr * p.ldc + col);
            old[it] = (col_ok && rr < p.M) ? (cs ? __ldcs(src) : *src) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
          __syncwarp();  // the previous chunk's reads of the pad are done
#pragma unroll
          for (int v = 0; v < 8; v++)
            *reinterpret_cast<uint4*>(pad + lane * EPI_LD + v * 4) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const long long rr = row_base + it * 4 + sub_row;
            if (col_ok && rr < p.M) {
              const float4 a4 = *reinterpret_cast<const float4*>(pad + (it * 4 + sub_row) * EPI_LD + sub_col);
              float4 o;
              o.x = __fadd_rn(__fmul_rn(p.alpha, a4.x), __fmul_rn(beta, old[it].x));
              o.y = __fadd_rn(__fmul_rn(p.alpha, a4.y), __fmul_rn(beta, old[it].y));
              o.z = __fadd_rn(__fmul_rn(p.alpha, a4.z), __fmul_rn(beta, old[it].z));
              o.w = __fadd_rn(__fmul_rn(p.alpha, a4.w), __fmul_rn(beta, old[it].w));
              float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + rr * p.ldc + col);
              if (cs) __stcs(dst, o);
              else *dst = o;
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < chunks; c++) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = tile_col0 + c * 32;
        if (row_ok && col0 < col_end) {
          {
#pragma unroll
            for (int v = 0; v < 4; v++) {
              const int col = col0 + v * 8;
              if (col < col_end) {
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
      }
      tc_fence_before_sync();
      __syncwarp();
      if (flag != nullptr && w.part + 1 < p.split) {
        // this warp's rows of C are written: hand them to the next K range
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_u32(flag, p.epoch * 8u + static_cast<uint32_t>(w.part) + 1u);
      }
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------ teardown --------------------------------------
  __syncwarp();
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the peer may still read its shared memory or signal it
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// Hand-over words of the split-K tail, [bank][tile][cta][warp]; a launch uses bank
// epoch % FLAG_BANKS, so up to FLAG_BANKS launches may be in flight on one device.
__device__ uint32_t g_split_flags[FLAG_BANKS * FLAG_TILES * 2 * 4];
uint32_t* g_split_flags_addr[64] = {};
uint32_t g_epoch = 0;

template <bool ACC_F16, typename CT>
cudaError_t launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const Tc2Params& p, int sm_count,
                        cudaStream_t stream) {
  auto kern = gemm_tc2_kernel<ACC_F16, CT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return e;
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = sm_count / 2;
  const int units = p.split_first + (tiles - p.split_first) * (p.nsplit > 1 ? p.nsplit : p.split);
  const int grid = 2 * (units < pairs ? units : pairs);
  return launch_with_pdl(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tmA, tmB, p);
}

}  // namespace

// Pair-tile width: 256 columns unless N is narrower.  Narrower tiles that would
// fill the last wave better were measured slower (4096^3: 1150 TFLOP/s at 256 vs
// 1010 at 224 and 990 at 192): per k-block every CTA stages 16 KB of A whatever
// the width, so a narrow tile moves more operand bytes per MMA cycle.
int pick_pair_bn(int N) {
  const int up = (N + 15) / 16 * 16;
  return up < 256 ? up : 256;
}

int launch_gemm_tc_pair(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                        int K, float alpha, float beta, bool acc_f16, bool c_f16, int bn_override, int sm_count,
                        uint32_t* status, cudaStream_t stream, const char** err) {
  CUtensorMap tmA, tmB;
  if (!make_tmap_2d(&tmA, A, TMAP_F16, M, K, lda, BM, BK, TMAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tmB, B, TMAP_F16, K, N, ldb, BK, 64, TMAP_SWIZZLE_128B)) {
    *err = "cuTensorMapEncodeTiled failed (alignment or driver entry point)";
    return -1;
  }
  Tc2Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.bn = (bn_override >= 32 && bn_override <= 256 && bn_override % 16 == 0) ? bn_override
                                                                           : pick_pair_bn(N);
  p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (N + p.bn - 1) / p.bn;
  // a raster band keeps about 32 MB of A rows hot in L2 while the B panels stream past
  long long g = (32ll << 20) / (2ll * BM * static_cast<long long>(K) * 2);
  p.group_m = static_cast<int>(g < 1 ? 1 : (g > 16 ? 16 : g));
  if (const char* gv = getenv("PHOBOS_GEMM_GROUP_M")) {   // tuning knob: row-blocks per raster band
    const int v = atoi(gv);
    if (v >= 1 && v <= 1024) p.group_m = v;
  }
  p.alpha = alpha;
  p.beta = beta;
  p.C = C;
  p.ldc = ldc;
  p.status = status;
  // split-K tail: when the last round would leave most CTA pairs idle, its tiles can be
  // cut into 2 or 4 K ranges that are added into C one after the other (f32 C only).
  // Off unless PHOBOS_GEMM_SPLITK=1: measured on 4096^3 it is no faster (1141 vs 1151
  // TFLOP/s), the K ranges of a tile serialise their epilogues at the very end.
  const int tiles = p.tiles_m * p.tiles_n, pairs = sm_count / 2;
  p.split = 1;
  p.split_first = tiles;
  p.flags = nullptr;
  p.epoch = 0;
  const int rem = tiles % pairs;
  const int num_kb = (K + BK - 1) / BK;
  const char* splitk = getenv("PHOBOS_GEMM_SPLITK");
  if (!c_f16 && tiles > pairs && rem > 0 && rem <= FLAG_TILES && 2 * rem <= pairs && splitk && splitk[0] == '1') {
    int split = (4 * rem <= pairs) ? 4 : 2;
    while (split > 1 && num_kb / split < 8) split >>= 1;
    int dev = 0;
    if (split > 1 && cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
      if (g_split_flags_addr[dev] == nullptr) {
        void* fp = nullptr;
        if (cudaGetSymbolAddress(&fp, g_split_flags) == cudaSuccess) g_split_flags_addr[dev] = static_cast<uint32_t*>(fp);
      }
      if (g_split_flags_addr[dev] != nullptr) {
        p.split = split;
        p.split_first = tiles - rem;
        p.flags = g_split_flags_addr[dev];
        p.epoch = __atomic_add_fetch(&g_epoch, 1u, __ATOMIC_RELAXED);
      }
    }
  }
  // split-N tail: with 256-wide tiles and a last round that fills at most half of the pairs, the last
  // round's tiles are computed as 128-wide halves (a 128-wide pair MMA takes ~122 clocks against ~171
  // for 256, so the round shrinks from 43.8 K to 31.2 K clocks at K = 4096).  PHOBOS_GEMM_NSPLIT=0 turns it off.
  p.nsplit = 1;
  {
    const char* ns = getenv("PHOBOS_GEMM_NSPLIT");
    const bool want = !(ns && ns[0] == '0');
    if (want && p.split == 1 && p.bn == 256 && tiles > pairs && rem > 0 && 2 * rem <= pairs && N % 256 == 0) {
      p.nsplit = 2;
      p.split_first = tiles - rem;
    }
  }
  // PHOBOS_GEMM_STREAMS=2 keeps two tiles of a pair in flight, each with its own producer,
  // issuer thread and accumulator (two issuing threads overlap their MMAs in an idle-SM
  // test: 151 against 171 clocks per 256-wide MMA).  Off by default: measured on the real
  // kernel it gains nothing at 8192^3 (1548 TFLOP/s either way) and loses at 4096^3
  // (1058 against 1150: with 3.46 tiles per pair the second stream only lengthens the tail).
  p.l2hint = 0;
  if (const char* hv = getenv("PHOBOS_GEMM_L2HINT")) p.l2hint = atoi(hv) & 7;
  p.streams = 1;
  if (const char* sv = getenv("PHOBOS_GEMM_STREAMS")) p.streams = (sv[0] == '2') ? 2 : 1;
  if (p.split > 1) p.streams = 1;  // the K ranges of a split tile must run one after the other
  cudaError_t e;
  if (!acc_f16 && !c_f16) {
    e = launch_pair<false, float>(tmA, tmB, p, sm_count, stream);
  } else if (acc_f16 && c_f16) {
    e = launch_pair<true, __half>(tmA, tmB, p, sm_count, stream);
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
