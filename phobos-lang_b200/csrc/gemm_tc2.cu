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
// Warp roles per CTA (320 threads): warp 0 TMA producer, warp 1 MMA issuer
// (leader CTA only) and tensor-memory owner, warps 2..9 epilogue
// (tcgen05.ld -> alpha*acc + beta*C_old -> global).  Two accumulator buffers of
// 256 columns let the epilogue of one work item overlap the main loop of the next.
// BN is a run-time multiple of 16 (<= 256): 256 unless N is narrower.
//
// Work distribution.  The kernel is persistent: CTA pair p of P works through a
// list of items.  Whole tiles are dealt round-robin (tile p, p + P, ...), in a
// raster of bands of `group_m` tile rows whose direction alternates from band to
// band, so that the A rows of a band and the B panels at the turn stay in L2.
// When the tile count is not a multiple of P the last round would leave pairs
// idle (4096^3: 256 tiles on 74 pairs = 3.46 rounds).  With a workspace from the
// caller, the last full round and the remainder are therefore shared out stream-K
// style: each of these tiles is cut along K into g equal pieces, and the pieces, laid
// end to end, are dealt to the P pairs as evenly as whole pieces go (4096^3: halves,
// three per pair, 1.5 tiles instead of 2).  Pieces are never shorter than 24 k-blocks:
// an epilogue takes about as long as 27 k-blocks of MMAs and there are two accumulator
// buffers, so shorter items would make the MMA issuer wait for the epilogue warps
// (measured: 107 us with ranges cut anywhere, against 104 us without sharing).  A range
// is at least one tile long, so a tile is shared by at most two pairs: the pair
// whose range ENDS inside the tile computes its first k-blocks (as the last item
// of its list) and the pair whose range STARTS inside it the rest (as the first
// item of its stream-K part).  The latter dumps its raw accumulator into the
// workspace early and raises a flag; the former, arriving at the very end,
// adds that partial to its own accumulator and runs the one epilogue of the
// tile.  Every output element is thus written exactly once, and no pair ever
// waits for work that has not long been finished.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int BM = 128;       // rows per CTA; 256 per pair
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 320;
constexpr int EPI_WARP0 = 2;  // warps 2..9: TMEM lane quarter = warp & 3 -> 2, 3, 0, 1, 2, 3, 0, 1
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_BYTES = BK * 128 * 2;         // 16 KB: up to 128 columns (two 64-column boxes) per CTA
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 8 * 32 * 32 * 4;    // one swizzled 32 x 32 f32 transpose pad per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256;               // tensor-memory columns per accumulator buffer
constexpr int SK_MIN_PIECE = 24;              // k-blocks: no shared tile is cut into pieces shorter than this
constexpr int SK_SLOT_WORDS = 2 * 4 * 32 * 256;  // one partial tile: [cta][warp][column][lane] 32-bit words
constexpr int FLAG_BANKS = 8;                 // launches that may be in flight per device
constexpr int MAX_PAIRS = 128;

enum ItemRole : int { ROLE_FULL = 0, ROLE_DUMP = 1, ROLE_FIXUP = 2 };

struct Tc2Params {
  int M, N, K;
  int bn;                 // N extent of a pair tile
  int tiles_m, tiles_n;   // pair tiles
  int group_m;            // tile rows per raster band
  float alpha, beta;
  void* C;
  long long ldc;
  uint32_t* status;
  // stream-K part: tiles [dp_tiles, dp_tiles + sk_tiles) are shared out by k-blocks
  int dp_tiles;
  int sk_tiles;           // 0: every tile is computed whole by one pair
  int sk_g;               // pieces per shared tile
  // Start of every pair's range of the shared tiles, in k-blocks from the first shared tile (entry `pairs` is the
  // end).  The shared tiles are cut into sk_g equal pieces each and the pieces are dealt out as evenly as whole
  // pieces go, so a range starts and ends on piece boundaries and every item is at least a piece long.  Worked
  // out on the host: the device would spend a microsecond of 64-bit divisions on it between two items.
  int sk_bound[MAX_PAIRS + 1];
  uint32_t* partials;     // workspace: slot b (boundary between pair b-1 and pair b) at b * SK_SLOT_WORDS
  uint32_t* flags;        // [bank][boundary][cta][quarter][parity], raised to `epoch` when a partial is complete
  uint32_t epoch;
};

struct Item {
  int tile, kb0, kb1, role, slot;
};

// Item n of pair `pair`'s list; false when the list has ended.
__device__ __forceinline__ bool work_item(const Tc2Params& p, int pair, int num_pairs, int num_kb, int n, Item& w) {
  const int n_dp = pair < p.dp_tiles ? (p.dp_tiles - pair + num_pairs - 1) / num_pairs : 0;
  if (n < n_dp) {
    w.tile = pair + n * num_pairs;
    w.kb0 = 0;
    w.kb1 = num_kb;
    w.role = ROLE_FULL;
    w.slot = 0;
    return true;
  }
  if (p.sk_tiles == 0) return false;
  const int s = p.sk_bound[pair], e = p.sk_bound[pair + 1];
  const int t = s / num_kb + (n - n_dp);
  const int ps = max(s, t * num_kb), pe = min(e, (t + 1) * num_kb);
  if (ps >= pe) return false;
  w.tile = p.dp_tiles + t;
  w.kb0 = ps - t * num_kb;
  w.kb1 = pe - t * num_kb;
  if (w.kb0 == 0 && w.kb1 == num_kb) {
    w.role = ROLE_FULL;
    w.slot = 0;
  } else if (w.kb0 > 0) {   // the range starts inside this tile: the rest of the tile, handed over
    w.role = ROLE_DUMP;
    w.slot = pair;
  } else {                  // the range ends inside this tile: its first k-blocks, plus the epilogue
    w.role = ROLE_FIXUP;
    w.slot = pair + 1;
  }
  return true;
}

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Tile index -> (row block, column block): bands of group_m tile rows, walked column by column with the
// row index fastest; odd bands run right to left, so the B panels at the turn are still in L2.
__device__ __forceinline__ void pair_tile_coords(int t, const Tc2Params& p, int& mb, int& nb) {
  const int per_group = p.group_m * p.tiles_n;
  const int g = t / per_group;
  const int first_m = g * p.group_m;
  const int gsize = min(p.group_m, p.tiles_m - first_m);
  const int r = t - g * per_group;
  mb = first_m + r % gsize;
  nb = r / gsize;
  if (g & 1) nb = p.tiles_n - 1 - nb;
}

template <bool ACC_F16, typename CT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ Tc2Params p) {
  extern __shared__ uint8_t smem_raw[];
  // rounded up to 1024 B as an offset into the array: a pointer rebuilt from an integer would lose the
  // shared address space and turn every access through it into a generic load or store
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                       // used in the leader CTA
  uint64_t* empty = bars + STAGES;             // one per CTA
  uint64_t* tmem_full = bars + 2 * STAGES;     // one per CTA
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // used in the leader CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  unsigned long long* clock_slot = reinterpret_cast<unsigned long long*>(bars + 2 * STAGES + 6);
  float* epi_pad = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const WaitCtx wctx{abort_flag, p.status};
  const bool clock_cta = threadIdx.x == 0 && blockIdx.x == 0;
  if (clock_cta) launch_clock_begin(clock_slot);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], 16);  // eight epilogue warps in each CTA of the pair
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

  const int num_kb = (p.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) --------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Item w;
      for (int n = 0; ok && work_item(p, pair, num_pairs, num_kb, n, w); n++) {
        int mb, nb;
        pair_tile_coords(w.tile, p, mb, nb);
        const int row0 = mb * (2 * BM) + static_cast<int>(rank) * BM;
        const int half_n = p.bn >> 1;                 // B columns staged by each CTA
        const int nbox = (half_n + 63) >> 6;
        const uint32_t stage_tx = 2u * static_cast<uint32_t>(A_BYTES + nbox * (BK * 128));
        const int col0 = nb * p.bn + static_cast<int>(rank) * half_n;
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          if (!mbar_wait(&empty[stage], phase ^ 1, SITE_GEMM_PRODUCER_EMPTY, wctx)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_u32(smem_u32(&full[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&full[stage], stage_tx);  // bytes of both CTAs' loads
          tma_load_2d_pair(sA + stage * A_BYTES, &tmA, full_leader, kb * BK, row0);
          for (int j = 0; j < nbox; j++)
            tma_load_2d_pair(sB + stage * B_BYTES + j * (BK * 128), &tmB, full_leader, col0 + j * 64, kb * BK);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA) ----------------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t idesc = umma_idesc_f16(2 * BM, p.bn, !ACC_F16, /*a_mn=*/false, /*b_mn=*/true);
      Item w;
      for (int n = 0; ok && work_item(p, pair, num_pairs, num_kb, n, w); n++) {
        const int acc = n & 1;
        const uint32_t acc_phase = (n >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, SITE_GEMM_MMA_TMEM_EMPTY, wctx)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          if (!mbar_wait(&full[stage], phase, SITE_GEMM_MMA_FULL, wctx)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            const uint64_t a_desc = umma_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = umma_smem_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024);
            umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb != w.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 0x3);  // both CTAs may refill this stage
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 0x3);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ---------------------------
    // Eight warps: two per tensor-memory lane quarter (a warp may only read the quarter warp % 4), each taking
    // every other 32-column chunk of its 32 rows.  The time of an epilogue is a chain of global-memory round
    // trips (C_old of a chunk must arrive before the chunk can be written), one per chunk: splitting the chunks
    // over two warps and requesting a warp's next C_old chunk before it works on the current one cut the chain
    // from eight exposed round trips to about two.
    const int q = warp & 3;
    const int half = (warp - EPI_WARP0) >> 2;   // 0: even chunks, 1: odd chunks
    int acc = 0;
    uint32_t acc_phase = 0;
    Item w;
    for (int n = 0; work_item(p, pair, num_pairs, num_kb, n, w); n++) {
      int mb, nb;
      pair_tile_coords(w.tile, p, mb, nb);
      if (!PH_WARP_WAIT(&tmem_full[acc], acc_phase, SITE_GEMM_EPI_TMEM_FULL, wctx)) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * ACC_STRIDE;
      const int chunks = (p.bn + 31) >> 5;
      // this quarter's part of a partial tile: [column][lane], so that a warp instruction moves 128 contiguous bytes
      uint32_t* part = p.partials + static_cast<size_t>(w.slot) * SK_SLOT_WORDS +
                       static_cast<size_t>((rank * 4 + q) * 256) * 32 + lane;
      uint32_t* flag = p.flags + ((((p.epoch % FLAG_BANKS) * 128 + w.slot) * 2 + rank) * 4 + q) * 2 + half;
      if (w.role == ROLE_DUMP) {
#pragma unroll 1
        for (int c = half; c < chunks; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 32; v++) part[(c * 32 + v) * 32] = r[v];
        }
        tc_fence_before_sync();
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          st_release_u32(flag, p.epoch);
          mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
        continue;
      }
      const bool fixup = w.role == ROLE_FIXUP;
      if (fixup) {
        // the other part of this tile was dumped at the start of its pair's stream-K range
        uint32_t okw = 1;
        if (lane == 0) {
          const uint64_t t0 = globaltimer_ns();
          while (ld_acquire_u32(flag) != p.epoch) {
            if (*abort_flag != 0 || globaltimer_ns() - t0 > wctx.limit_ns) {
              okw = 0;
              *abort_flag = SITE_GEMM_FIXUP_FLAG;
              atomicCAS(p.status, 0u, SITE_GEMM_FIXUP_FLAG | (blockIdx.x << 8));
              break;
            }
          }
        }
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) break;
      }
      const int row = mb * (2 * BM) + static_cast<int>(rank) * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      CT* crow = reinterpret_cast<CT*>(p.C) + static_cast<long long>(row) * p.ldc;
      const int tile_col0 = nb * p.bn;
      const int col_end = min(p.N, tile_col0 + p.bn);
      // the other pair's partial of the chunk in hand, requested one chunk ahead of its use
      uint32_t pcur[32];
      if (fixup && half < chunks) {
#pragma unroll
        for (int v = 0; v < 32; v++) pcur[v] = __ldcg(part + (half * 32 + v) * 32);
      }
      if constexpr (sizeof(CT) == 4) {
        // f32 C.  The accumulator arrives one row per lane; going to global memory that
        // way makes every warp instruction touch 32 different rows (16 useful bytes per
        // 32-byte sector, poor DRAM locality).  Each 32x32 chunk is therefore transposed
        // through a per-warp shared-memory pad (16-byte groups XOR-swizzled by row, so both
        // directions run at four wavefronts per 512 bytes) and a warp instruction covers
        // 4 rows x 128 contiguous bytes of C.
        float* pad = epi_pad + (warp - EPI_WARP0) * (32 * 32);
        const int sub_row = lane >> 3, grp = lane & 7, sub_col = grp * 4;
        const long long row_base = static_cast<long long>(mb) * (2 * BM) + static_cast<int>(rank) * BM + q * 32;
        auto load_old = [&](int c, float4 (&dst)[8]) {
          const int col = tile_col0 + c * 32 + sub_col;
          const bool col_ok = c < chunks && col < col_end;
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const long long rr = row_base + it * 4 + sub_row;
            const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.C) + rr * p.ldc + col);
            dst[it] = (col_ok && rr < p.M) ? *src : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        };
        float4 old[8];
        load_old(half, old);
#pragma unroll 1
        for (int c = half; c < chunks; c += 2) {
          const int col = tile_col0 + c * 32 + sub_col;
          const bool col_ok = col < col_end;
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
          if (fixup) {
#pragma unroll
            for (int v = 0; v < 32; v++) r[v] = __float_as_uint(__uint_as_float(r[v]) + __uint_as_float(pcur[v]));
            if (c + 2 < chunks) {   // the registers are free again: request this warp's next chunk of the partial
#pragma unroll
              for (int v = 0; v < 32; v++) pcur[v] = __ldcg(part + ((c + 2) * 32 + v) * 32);
            }
          }
          __syncwarp();  // the previous chunk's reads of the pad are done
#pragma unroll
          for (int v = 0; v < 8; v++)
            *reinterpret_cast<uint4*>(pad + lane * 32 + ((v ^ (lane & 7)) << 2)) =
                make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int pr = it * 4 + sub_row;
            const long long rr = row_base + pr;
            if (col_ok && rr < p.M) {
              const float4 a4 = *reinterpret_cast<const float4*>(pad + pr * 32 + ((grp ^ (pr & 7)) << 2));
              float4 o;
              o.x = __fadd_rn(__fmul_rn(p.alpha, a4.x), __fmul_rn(p.beta, old[it].x));
              o.y = __fadd_rn(__fmul_rn(p.alpha, a4.y), __fmul_rn(p.beta, old[it].y));
              o.z = __fadd_rn(__fmul_rn(p.alpha, a4.z), __fmul_rn(p.beta, old[it].z));
              o.w = __fadd_rn(__fmul_rn(p.alpha, a4.w), __fmul_rn(p.beta, old[it].w));
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + rr * p.ldc + col) = o;
            }
          }
          load_old(c + 2, old);   // in flight while the next chunk's accumulator is fetched and transposed
        }
      } else {
        // f16 C: one row per lane, 64 bytes of the row per chunk; the next chunk's C_old is requested ahead
        auto load_old = [&](int c, uint4 (&dst)[4]) {
          const int col0 = tile_col0 + c * 32;
#pragma unroll
          for (int v = 0; v < 4; v++) {
            const int col = col0 + v * 8;
            dst[v] = (row_ok && c < chunks && col < col_end) ? *reinterpret_cast<const uint4*>(crow + col)
                                                              : make_uint4(0u, 0u, 0u, 0u);
          }
        };
        uint4 old[4];
        load_old(half, old);
#pragma unroll 1
        for (int c = half; c < chunks; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
          float accv[32];
#pragma unroll
          for (int v = 0; v < 32; v++) {
            if constexpr (ACC_F16) accv[v] = __half2float(__ushort_as_half(static_cast<unsigned short>(r[v] & 0xFFFF)));
            else accv[v] = __uint_as_float(r[v]);
          }
          if (fixup) {
            // the two parts of the f16 accumulation are added in f32
#pragma unroll
            for (int v = 0; v < 32; v++) {
              if constexpr (ACC_F16) accv[v] += __half2float(__ushort_as_half(static_cast<unsigned short>(pcur[v] & 0xFFFF)));
              else accv[v] += __uint_as_float(pcur[v]);
            }
            if (c + 2 < chunks) {
#pragma unroll
              for (int v = 0; v < 32; v++) pcur[v] = __ldcg(part + ((c + 2) * 32 + v) * 32);
            }
          }
          const int col0 = tile_col0 + c * 32;
          if (row_ok && col0 < col_end) {
#pragma unroll
            for (int v = 0; v < 4; v++) {
              const int col = col0 + v * 8;
              if (col < col_end) {
                const __half2* oh = reinterpret_cast<const __half2*>(&old[v]);
                uint4 outv;
                __half2* outh = reinterpret_cast<__half2*>(&outv);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                  const float2 of = __half22float2(oh[e]);
                  const float x = __fadd_rn(__fmul_rn(p.alpha, accv[v * 8 + 2 * e]), __fmul_rn(p.beta, of.x));
                  const float y = __fadd_rn(__fmul_rn(p.alpha, accv[v * 8 + 2 * e + 1]), __fmul_rn(p.beta, of.y));
                  outh[e] = __floats2half2_rn(x, y);
                }
                *reinterpret_cast<uint4*>(crow + col) = outv;
              }
            }
          }
          load_old(c + 2, old);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
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
  if (clock_cta) launch_clock_end(clock_slot, p.status);
}

// Flags of the stream-K hand-over, [bank][boundary < 128][cta][lane quarter][chunk parity]; a launch uses bank epoch % FLAG_BANKS and
// the value `epoch`, so up to FLAG_BANKS launches may be in flight on one device without clearing anything.
__device__ uint32_t g_sk_flags[FLAG_BANKS * 128 * 2 * 4 * 2];
uint32_t* g_sk_flags_addr[64] = {};
uint32_t g_epoch = 0;

template <bool ACC_F16, typename CT>
cudaError_t launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const Tc2Params& p, int pairs,
                        cudaStream_t stream) {
  auto kern = gemm_tc2_kernel<ACC_F16, CT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return e;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  return launch_with_pdl(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tmA, tmB, p);
}

}  // namespace

// Pair-tile width: 256 columns unless N is narrower.  Narrower tiles that would
// fill the last round better were measured slower (4096^3: 1150 TFLOP/s at 256 vs
// 1010 at 224 and 990 at 192): per k-block every CTA stages 16 KB of A whatever
// the width, so a narrow tile moves more operand bytes per MMA cycle.
int pick_pair_bn(int N) {
  const int up = (N + 15) / 16 * 16;
  return up < 256 ? up : 256;
}

// Pieces per shared tile that minimise the work of the busiest pair when the last full round and the remainder
// (`shared` tiles on `pairs` pairs) are dealt out in pieces; 1 means sharing gains nothing over whole tiles.
static int pick_sk_pieces(long long shared, int pairs, int num_kb) {
  int best_g = 1;
  double best = static_cast<double>((shared + pairs - 1) / pairs);   // whole tiles: rounds
  for (int g = 2; g <= 8 && num_kb / g >= SK_MIN_PIECE; g++) {
    const double load = static_cast<double>((shared * g + pairs - 1) / pairs) / g;
    if (load < best - 0.05) {   // a gain under 5% of a tile does not pay for the partial tiles
      best = load;
      best_g = g;
    }
  }
  return best_g;
}

// Workspace that lets the pair kernel share out its last rounds stream-K style: one partial tile per pair boundary.
// 0 when the kernel would not use one for this problem.
size_t gemm_tc_pair_workspace_bytes(int M, int N, int K, int sm_count) {
  const int pairs = sm_count / 2;
  const int bn = pick_pair_bn(N);
  const long long tiles = static_cast<long long>((M + 2 * BM - 1) / (2 * BM)) * ((N + bn - 1) / bn);
  const int num_kb = (K + BK - 1) / BK;
  if (pairs < 2 || pairs > MAX_PAIRS || tiles < pairs || tiles % pairs == 0) return 0;
  if (tiles * num_kb > 0x3fffffffLL) return 0;   // ranges are kept in 32-bit k-block counts
  if (pick_sk_pieces(pairs + tiles % pairs, pairs, num_kb) == 1) return 0;
  return static_cast<size_t>(pairs) * SK_SLOT_WORDS * 4;
}

int launch_gemm_tc_pair(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                        int K, float alpha, float beta, bool acc_f16, bool c_f16, int sm_count, void* workspace,
                        size_t workspace_bytes, uint32_t* status, cudaStream_t stream, const char** err) {
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
  p.bn = pick_pair_bn(N);
  p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (N + p.bn - 1) / p.bn;
  // a raster band keeps about 32 MB of A rows hot in L2 while the B panels stream past
  // (measured at 8192^3 f16: 8 tile rows is the best of 2 / 4 / 8 / 16 / 32)
  long long g = (32ll << 20) / (2ll * BM * static_cast<long long>(K) * 2);
  p.group_m = static_cast<int>(g < 1 ? 1 : (g > 16 ? 16 : g));
  p.alpha = alpha;
  p.beta = beta;
  p.C = C;
  p.ldc = ldc;
  p.status = status;
  const int tiles = p.tiles_m * p.tiles_n, pairs = sm_count / 2;
  p.dp_tiles = tiles;
  p.sk_tiles = 0;
  p.sk_g = 1;
  const size_t need = gemm_tc_pair_workspace_bytes(M, N, K, sm_count);
  int dev = 0;
  if (need > 0 && workspace != nullptr && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 256 == 0 &&
      cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    if (g_sk_flags_addr[dev] == nullptr) {
      void* fp = nullptr;
      if (cudaGetSymbolAddress(&fp, g_sk_flags) == cudaSuccess) g_sk_flags_addr[dev] = static_cast<uint32_t*>(fp);
    }
    if (g_sk_flags_addr[dev] != nullptr) {
      // the last full round and the remainder are shared out in pieces
      p.dp_tiles = (tiles / pairs - 1) * pairs;
      p.sk_tiles = tiles - p.dp_tiles;
      const int num_kb = (K + BK - 1) / BK;
      p.sk_g = pick_sk_pieces(p.sk_tiles, pairs, num_kb);
      const long long units = static_cast<long long>(p.sk_tiles) * p.sk_g;
      for (int i = 0; i <= pairs; i++) {
        const long long ub = units * i / pairs;
        p.sk_bound[i] = static_cast<int>((ub / p.sk_g) * num_kb + (ub % p.sk_g) * num_kb / p.sk_g);
      }
      p.partials = static_cast<uint32_t*>(workspace);
      p.flags = g_sk_flags_addr[dev];
      uint32_t ep = __atomic_add_fetch(&g_epoch, 1u, __ATOMIC_RELAXED);
      if (ep == 0) ep = __atomic_add_fetch(&g_epoch, 1u, __ATOMIC_RELAXED);  // 0 is what untouched flags hold
      p.epoch = ep;
    }
  }
  cudaError_t e;
  if (!acc_f16 && !c_f16) {
    e = launch_pair<false, float>(tmA, tmB, p, pairs, stream);
  } else if (acc_f16 && c_f16) {
    e = launch_pair<true, __half>(tmA, tmB, p, pairs, stream);
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
