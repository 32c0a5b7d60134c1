// Flash attention forward (non-causal) for sm_100a.
//
// Covers the reference's `flash_attention` kernels
// (examples/flash_attention_fp16.ph:1-50, flash_attention_fp32.ph:1-45; device
// code emitted by emit_frag_for, phobos-lang/src/codegen/frag.rs:488-583).  The
// recurrence per query row, streaming over key blocks, is the reference's:
//   s = (q . k) * scale          f16 x f16 products, f32 accumulate, scale in f32
//   mnew = max(m, rowmax(s));  p = exp(s - mnew)   via ex2.approx.ftz, as
//                              phobos-lang/src/codegen/tile.rs:1033-1061
//   l = l*corr + rowsum(p)     over the unrounded f32 p
//   acc = acc*corr + f16(p) @ v     P rounded RN to f16 for the MMA (frag.rs:384-432)
//   O = acc / l                rounded RN to f16 on store (frag.rs:437-454)
// with one difference that leaves the result unchanged up to rounding: the
// rescale by corr is applied only when the running maximum grew by more than
// 2^8 (the stale maximum is kept otherwise; O and l stay consistent, and
// O = acc / l cancels the common factor).
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles that
// ping-pong so that the tensor core works on one tile while the other tile's
// softmax runs.  Warp roles (320 threads):
//   warps 0-3  softmax + correction + epilogue of query tile 0 (one row per thread)
//   warps 4-7  the same for query tile 1
//   warp 8     TMA producer: Q once, then K and V blocks of 128 keys, 2 stages each
//   warp 9     tcgen05.mma issuer: S_i = Q_i K^T into tensor memory, then
//              O_i += P_i V with P_i read from tensor memory (it overwrites S_i)
// Tensor memory columns: S0 | S1 | O0 | O1.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int QT = 128;        // query rows per tile
constexpr int KB = 128;        // keys per block
constexpr int FL_THREADS = 320;
constexpr float RESCALE_TAU = 8.0f;          // log2 units
constexpr float M_INIT = -65504.0f * 1.4426950408889634f;  // the .ph's -65504 in log2 units

template <int D>
struct FCfg {
  static constexpr int HALVES = D / 64;               // 128-byte swizzle atoms along the head dim
  static constexpr int QTILE_BYTES = QT * D * 2;
  static constexpr int KV_BYTES = KB * D * 2;
  static constexpr int HALF_BYTES = 128 * 128;        // one [128 rows x 64 f16] box
  static constexpr int SMEM_BYTES = 2 * QTILE_BYTES + 4 * KV_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int S_COL0 = 0;                    // S_i at i*128
  static constexpr int O_COL0 = 256;                  // O_i at 256 + i*D
};

struct FlashParams {
  int Nq, Nk;
  int n_kblocks;
  float scale_log2;   // |scale| * log2(e)
  int negate_q;       // scale < 0: negate Q inside the MMA instead
  void* O;            // [BH][Nq][D]
  uint32_t* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int D, bool OUT_F32>
__global__ void __launch_bounds__(FL_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FlashParams p) {
  using C_ = FCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // 2 tiles
  uint8_t* sK = smem + 2 * C_::QTILE_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * C_::KV_BYTES;                 // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * C_::KV_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2 (per query tile)
  uint64_t* p_full = bars + 11;     // 2
  uint64_t* o_done = bars + 13;     // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wctx{abort_flag, p.status};
  const int head = blockIdx.y;
  const int q_row0 = blockIdx.x * (2 * QT);
  const int nkb = p.n_kblocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&o_done[s], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * C_::QTILE_BYTES);
      for (int i = 0; i < 2; i++)
        for (int h = 0; h < C_::HALVES; h++)
          tma_load_3d(sQ + i * C_::QTILE_BYTES + h * C_::HALF_BYTES, &tmQ, q_full, h * 64, q_row0 + i * QT, head);
      for (int j = 0; j < nkb; j++) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par, SITE_FLASH_LOAD, wctx)) break;
        mbar_arrive_expect_tx(&k_full[st], C_::KV_BYTES);
        for (int h = 0; h < C_::HALVES; h++)
          tma_load_3d(sK + st * C_::KV_BYTES + h * C_::HALF_BYTES, &tmK, &k_full[st], h * 64, j * KB, head);
        if (!mbar_wait(&v_empty[st], par, SITE_FLASH_LOAD, wctx)) break;
        mbar_arrive_expect_tx(&v_full[st], C_::KV_BYTES);
        for (int h = 0; h < C_::HALVES; h++)
          tma_load_3d(sV + st * C_::KV_BYTES + h * C_::HALF_BYTES, &tmV, &v_full[st], h * 64, j * KB, head);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      // S = Q K^T : M=128 (queries), N=128 (keys), both operands K-major
      const uint32_t idesc_s = umma_idesc_f16(QT, KB, true, false, false) | (p.negate_q ? (1u << 13) : 0u);
      // O += P V : M=128, N=D, A (P) from tensor memory, B (V) N-major
      constexpr uint32_t idesc_o = umma_idesc_f16(QT, D, true, false, true);
      auto issue_s = [&](int i, int kstage) {
        const uint32_t qa = smem_u32(sQ + i * C_::QTILE_BYTES);
        const uint32_t ka = smem_u32(sK + kstage * C_::KV_BYTES);
        const uint32_t d = tmem_base + C_::S_COL0 + i * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
          const uint32_t off = (kk >> 2) * C_::HALF_BYTES + (kk & 3) * 32;
          umma_f16_ss(d, umma_smem_desc(qa + off, 16, 1024), umma_smem_desc(ka + off, 16, 1024), idesc_s,
                      kk != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int i, int vstage, bool accumulate) {
        const uint32_t va = smem_u32(sV + vstage * C_::KV_BYTES);
        const uint32_t d = tmem_base + C_::O_COL0 + i * D;
        const uint32_t pa = tmem_base + C_::S_COL0 + i * 128;  // P overwrote S, 2 f16 per column
#pragma unroll
        for (int kk = 0; kk < KB / 16; kk++) {
          // V block: [128 keys][64 d] per half; 8-key atoms 1024 B apart, halves HALF_BYTES apart
          umma_f16_ts(d, pa + kk * 8, umma_smem_desc(va + kk * 2048, C_::HALF_BYTES, 1024), idesc_o,
                      (accumulate || kk != 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(q_full, 0, SITE_FLASH_MMA, wctx) && mbar_wait(&k_full[0], 0, SITE_FLASH_MMA, wctx);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0, 0);
        umma_commit(&s_full[0]);
        issue_s(1, 0);
        umma_commit(&s_full[1]);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < nkb && ok; j++) {
        const int st = j & 1;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1, SITE_FLASH_MMA, wctx)) break;
        for (int i = 0; i < 2; i++) {
          if (!mbar_wait(&p_full[i], j & 1, SITE_FLASH_MMA, wctx)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_pv(i, st, j > 0);
          if (i == 1) umma_commit(&v_empty[st]);
          if (j + 1 < nkb) {
            const int ns = (j + 1) & 1;
            if (i == 0 && !mbar_wait(&k_full[ns], ((j + 1) >> 1) & 1, SITE_FLASH_MMA, wctx)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_s(i, ns);
            umma_commit(&s_full[i]);
            if (i == 1) umma_commit(&k_empty[ns]);
          } else {
            umma_commit(&o_done[i]);
          }
        }
      }
    }
  } else {
    // ------------------------------ softmax / correction / epilogue ---------------
    const int i = warp >> 2;       // query tile
    const int q = warp & 3;        // TMEM lane quarter
    const int row_in_tile = q * 32 + lane;
    const long long row = static_cast<long long>(q_row0) + i * QT + row_in_tile;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t s_addr = lane_base + C_::S_COL0 + i * 128;
    const uint32_t o_addr = lane_base + C_::O_COL0 + i * D;
    const float c = p.scale_log2;
    float m2 = M_INIT, l = 0.0f;
    bool ok = true;

    for (int j = 0; j < nkb; j++) {
      // the vote keeps the warp together: the TMEM loads below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[i], j & 1, SITE_FLASH_SOFTMAX, wctx))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t sr[4][32];
#pragma unroll
      for (int cc = 0; cc < 4; cc++) tmem_ld_32x32b_x32(s_addr + cc * 32, sr[cc]);
      tmem_ld_wait();
      const int valid = p.Nk - j * KB;  // keys of this block that exist
      if (valid < KB) {
#pragma unroll
        for (int cc = 0; cc < 4; cc++)
#pragma unroll
          for (int e = 0; e < 32; e++)
            if (cc * 32 + e >= valid) sr[cc][e] = 0xFF800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; e++) {
        mx0 = fmaxf(mx0, __uint_as_float(sr[0][e]));
        mx1 = fmaxf(mx1, __uint_as_float(sr[1][e]));
        mx2 = fmaxf(mx2, __uint_as_float(sr[2][e]));
        mx3 = fmaxf(mx3, __uint_as_float(sr[3][e]));
      }
      const float mnew = fmaxf(m2, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * c);
      if (j == 0) {
        m2 = mnew;  // O is not yet written: nothing to rescale
      } else {
        const bool need = (mnew - m2) > RESCALE_TAU;
        if (__any_sync(0xffffffffu, need)) {
          // S_i of block j is complete, so O_i += P V of block j-1 is complete too
          // (same issuing thread, in order): O_i may be rescaled in place.
          const float f = need ? ex2_approx(m2 - mnew) : 1.0f;
#pragma unroll 1
          for (int cc = 0; cc < D / 32; cc++) {
            uint32_t orr[32];
            tmem_ld_32x32b_x32(o_addr + cc * 32, orr);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e++) orr[e] = __float_as_uint(__uint_as_float(orr[e]) * f);
            tmem_st_32x32b_x32(o_addr + cc * 32, orr);
          }
          tmem_st_wait();
          l *= f;
          if (need) m2 = mnew;
        }
      }
      const float neg_m = -m2;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      uint32_t pk[2][32];
#pragma unroll
      for (int cc = 0; cc < 4; cc++) {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(sr[cc][e]), c, neg_m));
          float p1 = ex2_approx(fmaf(__uint_as_float(sr[cc][e + 1]), c, neg_m));
          if (valid < KB) {  // keys past the end contribute nothing
            if (cc * 32 + e >= valid) p0 = 0.0f;
            if (cc * 32 + e + 1 >= valid) p1 = 0.0f;
          }
          if ((e & 2) == 0) {
            l0 += p0;
            l1 += p1;
          } else {
            l2 += p0;
            l3 += p1;
          }
          pk[cc >> 1][(cc & 1) * 16 + (e >> 1)] = pack_f16x2(p0, p1);
        }
      }
      l += (l0 + l1) + (l2 + l3);
      tmem_st_32x32b_x32(s_addr, pk[0]);
      tmem_st_32x32b_x32(s_addr + 32, pk[1]);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_full[i]);
    }

    if (ok && __all_sync(0xffffffffu, mbar_wait(&o_done[i], 0, SITE_FLASH_EPI, wctx))) {
      tc_fence_after_sync();
      const float inv_l = 1.0f / l;
      const bool row_ok = row < p.Nq;
#pragma unroll 1
      for (int cc = 0; cc < D / 32; cc++) {
        uint32_t orr[32];
        tmem_ld_32x32b_x32(o_addr + cc * 32, orr);
        tmem_ld_wait();
        if (row_ok) {
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.O) + (static_cast<long long>(head) * p.Nq + row) * D + cc * 32;
#pragma unroll
            for (int v = 0; v < 8; v++) {
              float4 o;
              o.x = __uint_as_float(orr[4 * v + 0]) * inv_l;
              o.y = __uint_as_float(orr[4 * v + 1]) * inv_l;
              o.z = __uint_as_float(orr[4 * v + 2]) * inv_l;
              o.w = __uint_as_float(orr[4 * v + 3]) * inv_l;
              reinterpret_cast<float4*>(dst)[v] = o;
            }
          } else {
            __half* dst = reinterpret_cast<__half*>(p.O) + (static_cast<long long>(head) * p.Nq + row) * D + cc * 32;
#pragma unroll
            for (int v = 0; v < 4; v++) {
              uint4 o;
              o.x = pack_f16x2(__uint_as_float(orr[8 * v + 0]) * inv_l, __uint_as_float(orr[8 * v + 1]) * inv_l);
              o.y = pack_f16x2(__uint_as_float(orr[8 * v + 2]) * inv_l, __uint_as_float(orr[8 * v + 3]) * inv_l);
              o.z = pack_f16x2(__uint_as_float(orr[8 * v + 4]) * inv_l, __uint_as_float(orr[8 * v + 5]) * inv_l);
              o.w = pack_f16x2(__uint_as_float(orr[8 * v + 6]) * inv_l, __uint_as_float(orr[8 * v + 7]) * inv_l);
              reinterpret_cast<uint4*>(dst)[v] = o;
            }
          }
        }
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
  tc_fence_after_sync();
  if (warp == 9) tmem_dealloc(tmem_base, C_::TMEM_COLS);
}

template <int D, bool OUT_F32>
cudaError_t launch_d(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FlashParams& p,
                     long long batch_heads, cudaStream_t stream) {
  using C_ = FCfg<D>;
  auto kern = flash_fwd_kernel<D, OUT_F32>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid((p.Nq + 2 * QT - 1) / (2 * QT), static_cast<unsigned>(batch_heads));
  kern<<<grid, FL_THREADS, C_::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError();
}

}  // namespace

int launch_flash_f16(const void* Q, const void* K, const void* V, void* O, int out_f32, long long batch_heads,
                     int Nq, int Nk, int D, float scale, int sm_count, uint32_t* status, cudaStream_t stream,
                     const char** err) {
  (void)sm_count;
  if (D != 64 && D != 128) {
    *err = "flash_attention: head dim must be 64 or 128";
    return -2;
  }
  if (batch_heads > 65535) {
    *err = "flash_attention: more than 65535 (batch*head) problems in one launch";
    return -2;
  }
  CUtensorMap tmQ, tmK, tmV;
  const long long q_pitch = static_cast<long long>(Nq) * D, k_pitch = static_cast<long long>(Nk) * D;
  if (!make_tmap_3d(&tmQ, Q, TMAP_F16, batch_heads, Nq, D, D, q_pitch, QT, 64, TMAP_SWIZZLE_128B) ||
      !make_tmap_3d(&tmK, K, TMAP_F16, batch_heads, Nk, D, D, k_pitch, KB, 64, TMAP_SWIZZLE_128B) ||
      !make_tmap_3d(&tmV, V, TMAP_F16, batch_heads, Nk, D, D, k_pitch, KB, 64, TMAP_SWIZZLE_128B)) {
    *err = "cuTensorMapEncodeTiled failed (alignment or driver entry point)";
    return -1;
  }
  FlashParams p{};
  p.Nq = Nq;
  p.Nk = Nk;
  p.n_kblocks = (Nk + KB - 1) / KB;
  p.scale_log2 = fabsf(scale) * 1.4426950408889634f;
  p.negate_q = scale < 0.0f ? 1 : 0;
  p.O = O;
  p.status = status;
  cudaError_t e;
  if (D == 128)
    e = out_f32 ? launch_d<128, true>(tmQ, tmK, tmV, p, batch_heads, stream)
                : launch_d<128, false>(tmQ, tmK, tmV, p, batch_heads, stream);
  else
    e = out_f32 ? launch_d<64, true>(tmQ, tmK, tmV, p, batch_heads, stream)
                : launch_d<64, false>(tmQ, tmK, tmV, p, batch_heads, stream);
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
