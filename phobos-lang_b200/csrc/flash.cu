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
// softmax runs.  Warp roles (384 threads; the two softmax warpgroups raise their
// register budget with setmaxnreg, the third warpgroup lowers its own):
//   warps 0-3  softmax + correction + epilogue of query tile 0 (one row per thread)
//   warps 4-7  the same for query tile 1
//   warp 8     TMA producer: Q once, then K and V blocks of 128 keys through one
//              ring of five slots (a block takes thousands of clocks to land while
//              the MMAs saturate shared memory, so the ring runs two blocks ahead)
//   warps 9,10 tcgen05.mma issuers, one per query tile: S_i = Q_i K^T into tensor
//              memory, then O_i += P_i V with P_i read from tensor memory (it
//              overwrites S_i).  They take strict turns, so the two tiles keep
//              ping-ponging, but each issuer does the barrier waits of its next
//              batch while the other one issues (a tcgen05.mma blocks its thread
//              until the pipe accepts it; two free-running issuers fell into
//              lockstep and were 20% slower)
//   warp 11    idle (completes the third warpgroup)
// Tensor memory columns: S0 | S1 | O0 | O1.
//
// Exponentials: a 128x128 score tile needs 16384 exp2; the MUFU unit delivers 16
// per clock per SM, i.e. 1024 clocks per tile, the same order as the tensor core's
// time for the tile's two MMAs, so the two units have to overlap: that is what the
// two-tile ping-pong is for.  The scale/subtract and the row sums use packed f32x2
// instructions to halve their issue slots.
//
// Measured and not adopted (B4 H32 S4096 D128, this structure at 1108 TFLOP/s), each verified
// against the oracle first:
//  * P handed over in slices, each with its own barrier, so that O += P V could start
//    before the block's softmax has finished, with one issuing thread for both tiles:
//    1043 / 1015 / 867 / 639 TFLOP/s for 1 / 2 / 4 / 8 slices; each hand-over costs a
//    tcgen05.wait::st of some hundred clocks in the softmax warps;
//  * the first half of P stored to tensor memory while the second half is computed
//    (1099), S fetched in two halves with the maximum of the first taken while the
//    second is on its way (1106), both (1089);
//  * one or two of every eight exponential pairs as a cubic on the FMA pipes
//    (2^x = 2^n p(f), relative error 7.5e-5, well inside f16): 1085 / 1074;
//  * key blocks of 64 with TWO S buffers per tile (64 + 64 columns, what fits beside O at
//    D = 128), so that S(n+2) is computed while the softmax works on block n: 997 with one
//    issuing thread per tile, 1087 with two (one for S = Q K^T, one for O += P V), 967 when
//    the tiles are also made to take turns at the exponentials.  Clock stamps of that
//    kernel: a thread needs 70-110 clocks per tcgen05.mma it issues whatever the shape, and
//    a 64-key block needs 12 of them where a 128-key block needs 16 for twice the keys; from
//    P(n) handed over to S(n+2) seen by the softmax warps takes 2440 clocks (250 until the
//    issuer sees P, 280 to issue four MMAs, 350 until the S issuer sees them complete, 550 to
//    issue eight, 1000 until the last has left the shared in-order pipe and the softmax warp
//    has woken); both tiles' exponentials fall into step and share the MUFU unit (1250 clocks
//    per 64 keys).
//  * ONE 128-row tile per CTA with THREE 128-key S buffers beside O (a persistent CTA walks its
//    tiles; separate issuing threads for S = Q K^T and O += P V; separate K and Q/V producers),
//    so that S(n+1), S(n+2) are computed while the softmax works on block n.  Four forms, all
//    parity-green: both warpgroups on every block, each thread taking 64 of its row's keys and
//    exchanging the row maximum through shared memory (917); the warpgroups on alternate blocks,
//    the reference maximum handed from block to block, dedicated epilogue warps (972; 1005 with
//    the hand-over in one tagged word; 951 with hardware-suspending waits); the column split
//    again with the softmax loop software pipelined two blocks deep (753).  Clock stamps: every
//    shared-memory round trip of a softmax warp (an mbarrier that has long completed, a flag
//    word) costs 300-500 clocks while S = Q K^T streams both operands from shared memory at the
//    full 128 B/clk, and those forms need two or three of them per block where this kernel needs
//    one; a block's buffer is held for softmax + 2400 clocks (P seen by the issuer, 8 MMAs, the
//    commit seen by the other issuer, 8 MMAs, S seen), so three buffers give a period of
//    (softmax + 2400) / 3 >= 1900 clocks per block, no better than the 1920 of this kernel.
//  * The keys 64-127 of S(j+1) issued by a second thread per tile as soon as the softmax warps hold
//    S(j) in registers (those columns carry no P), so that 8 + 8 half-width MMAs instead of 16 follow
//    P: 1076 against 1135 on the same GPU; an N = 64 MMA occupies the pipe for ~57 clocks where an
//    N = 128 one takes ~77, so two halves cost more than the whole.
//  * The exponential loop on its own (register data, idle SM): 1180 clocks per 128 keys for one
//    warp per scheduler, 1050 per block with two (the MUFU floor is 1024: 4096 ex2 per scheduler
//    at 4 per clock); with 2/8 or 3/8 of the pairs as a cubic on the FMA/ALU pipes 1080 and 920:
//    the polynomial costs nearly the issue slots and ALU cycles it saves in MUFU cycles.
// The loop is bound by the dependency chain of a tile, softmax(j) -> P -> O += P V and
// S(j+1) -> softmax(j+1) (S, P and O of both tiles fill the 512 tensor-memory columns
// at D = 128, so a 128-key S cannot be double buffered without giving up the second tile),
// with the exponentials of one warp per scheduler at the MUFU rate inside it.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr int QT = 128;        // query rows per tile
constexpr int KB = 128;        // keys per block
constexpr int FL_THREADS = 384;
constexpr float RESCALE_TAU = 8.0f;          // log2 units
constexpr float M_INIT = -65504.0f * 1.4426950408889634f;  // the .ph's -65504 in log2 units

template <int D>
struct FCfg {
  static constexpr int HALVES = D / 64;               // 128-byte swizzle atoms along the head dim
  static constexpr int QTILE_BYTES = QT * D * 2;
  static constexpr int KV_BYTES = KB * D * 2;
  static constexpr int HALF_BYTES = 128 * 128;        // one [128 rows x 64 f16] box
  static constexpr int RING = 5;                      // K/V blocks in flight (shared ring)
  static constexpr int SMEM_BYTES = 2 * QTILE_BYTES + RING * KV_BYTES + 1024 + 256;
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

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <int D, bool OUT_F32>
__global__ void __launch_bounds__(FL_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FlashParams p) {
  using C_ = FCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  // rounded up to 1024 B as an offset into the array: a pointer rebuilt from an integer would lose the
  // shared address space and turn every access through it into a generic load or store
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // K and V blocks share one ring of RING slots, filled in consumption order
  // K0 V0 K1 V1 ...: item n (K_j = 2j, V_j = 2j+1) lives in slot n % RING.
  constexpr int RING = C_::RING;
  uint8_t* sQ = smem;                                  // 2 tiles
  uint8_t* sKV = smem + 2 * C_::QTILE_BYTES;           // RING slots
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + RING * C_::KV_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // RING
  uint64_t* kv_empty = bars + 1 + RING;    // RING
  uint64_t* s_full = bars + 1 + 2 * RING;  // 2 (per query tile)
  uint64_t* p_full = s_full + 2;           // 2
  uint64_t* o_done = s_full + 4;           // 2
  uint64_t* turn = s_full + 6;             // 2 (issuer hand-off)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wctx{abort_flag, p.status};
  // one CTA in the middle of the grid reports the SM clock it saw
  __shared__ unsigned long long clock_slot[2];
  const bool clock_cta = threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == (gridDim.y >> 1);
  if (clock_cta) launch_clock_begin(clock_slot);
  const int head = blockIdx.y;
  const int q_row0 = blockIdx.x * (2 * QT);
  const int nkb = p.n_kblocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < RING; s++) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 2);  // released by both issuers
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);    // one arrival per softmax warp
      mbar_init(&o_done[s], 1);
      mbar_init(&turn[s], 1);
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

  if (warp >= 8) {
  // the third warpgroup hands registers to the softmax warpgroups
  asm volatile("setmaxnreg.dec.sync.aligned.u32 120;");
  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * C_::QTILE_BYTES);
      for (int i = 0; i < 2; i++)
        for (int h = 0; h < C_::HALVES; h++)
          tma_load_3d(sQ + i * C_::QTILE_BYTES + h * C_::HALF_BYTES, &tmQ, q_full, h * 64, q_row0 + i * QT, head);
      int slot = 0;
      uint32_t par = 1;  // parity that a never-used slot's `empty` barrier passes
      for (int n = 0; n < 2 * nkb; n++) {
        const int j = n >> 1;
        const bool is_v = (n & 1) != 0;
        if (!mbar_wait(&kv_empty[slot], par, SITE_FLASH_LOAD, wctx)) break;
        mbar_arrive_expect_tx(&kv_full[slot], C_::KV_BYTES);
        for (int h = 0; h < C_::HALVES; h++)
          tma_load_3d(sKV + slot * C_::KV_BYTES + h * C_::HALF_BYTES, is_v ? &tmV : &tmK, &kv_full[slot], h * 64,
                      j * KB, head);
        if (++slot == RING) {
          slot = 0;
          par ^= 1;
        }
      }
    }
  } else if (warp <= 10) {
    // ------------------------------ MMA issuers (warp 9: tile 0, warp 10: tile 1) ---
    if (lane == 0) {
      // S = Q K^T : M=128 (queries), N=128 (keys), both operands K-major
      const uint32_t idesc_s = umma_idesc_f16(QT, KB, true, false, false) | (p.negate_q ? (1u << 13) : 0u);
      // O += P V : M=128, N=D, A (P) from tensor memory, B (V) N-major
      constexpr uint32_t idesc_o = umma_idesc_f16(QT, D, true, false, true);
      // descriptors are built once; an operand elsewhere is the base descriptor plus
      // its byte offset >> 4 in the address field
      const uint64_t q_desc0 = umma_smem_desc(smem_u32(sQ), 16, 1024);                    // K-major
      const uint64_t k_desc0 = umma_smem_desc(smem_u32(sKV), 16, 1024);                   // K-major
      const uint64_t v_desc0 = umma_smem_desc(smem_u32(sKV), C_::HALF_BYTES, 1024);       // N-major
      auto issue_s = [&](int i, int slot) {
        const uint64_t qd = q_desc0 + static_cast<uint64_t>(i * (C_::QTILE_BYTES >> 4));
        const uint64_t kd = k_desc0 + static_cast<uint64_t>(slot * (C_::KV_BYTES >> 4));
        const uint32_t d = tmem_base + C_::S_COL0 + i * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * C_::HALF_BYTES + (kk & 3) * 32) >> 4);
          umma_f16_ss(d, qd + off, kd + off, idesc_s, kk != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int i, int slot, bool accumulate) {
        const uint64_t vd = v_desc0 + static_cast<uint64_t>(slot * (C_::KV_BYTES >> 4));
        const uint32_t d = tmem_base + C_::O_COL0 + i * D;
        const uint32_t pa = tmem_base + C_::S_COL0 + i * 128;  // P overwrote S, 2 f16 per column
#pragma unroll
        for (int kk = 0; kk < KB / 16; kk++) {
          // V block: [128 keys][64 d] per half; 8-key atoms 1024 B apart, halves HALF_BYTES apart;
          // a step of 16 keys is 2048 B
          umma_f16_ts(d, pa + kk * 8, vd + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_o,
                      (accumulate || kk != 0) ? 1u : 0u);
        }
      };
      // ring cursor, advanced once per item in consumption order K0 V0 K1 V1 ...
      int cur = 0;
      uint32_t cpar = 0;
      auto advance = [&]() {
        if (++cur == RING) {
          cur = 0;
          cpar ^= 1;
        }
      };
      // Issuer warp 9 owns query tile 0, warp 10 tile 1.  They take turns: while
      // one issues its 16 MMAs (each tcgen05.mma blocks its thread until the pipe
      // accepts it, ~96 clocks), the other performs the barrier waits of its next
      // batch, so the tensor pipe never idles behind a wait.  turn[t] is arrived by
      // the other issuer when its batch is issued.
      const int i = warp - 9;
      bool ok = mbar_wait(q_full, 0, SITE_FLASH_MMA, wctx) && mbar_wait(&kv_full[cur], cpar, SITE_FLASH_MMA, wctx);
      if (ok) {
        tc_fence_after_sync();
        issue_s(i, cur);
        umma_commit(&s_full[i]);
        umma_commit(&kv_empty[cur]);
        advance();
      }
      for (int j = 0; j < nkb && ok; j++) {
        const int vs = cur;
        if (!mbar_wait(&kv_full[vs], cpar, SITE_FLASH_MMA, wctx)) break;
        advance();
        const int ks = cur;
        const bool more = j + 1 < nkb;
        if (more) {
          if (!mbar_wait(&kv_full[ks], cpar, SITE_FLASH_MMA, wctx)) break;
          advance();
        }
        // my turn: tile 0 goes first in every round (its barrier passes once before any arrival)
        if (!mbar_wait(&turn[i], i == 0 ? ((j & 1) ^ 1) : (j & 1), SITE_FLASH_MMA, wctx)) break;
        // P_i is the late input: everything else has been waited for by now
        if (!mbar_wait(&p_full[i], j & 1, SITE_FLASH_MMA, wctx)) break;
        tc_fence_after_sync();
        issue_pv(i, vs, j > 0);
        umma_commit(&kv_empty[vs]);
        if (more) {
          issue_s(i, ks);
          umma_commit(&s_full[i]);
          umma_commit(&kv_empty[ks]);
        } else {
          umma_commit(&o_done[i]);
        }
        mbar_arrive(&turn[i ^ 1]);
      }
    }
  }
  } else {
    // ------------------------------ softmax / correction / epilogue ---------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
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
      if (!PH_WARP_WAIT(&s_full[i], j & 1, SITE_FLASH_SOFTMAX, wctx)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t sr[4][32];
      const int valid = p.Nk - j * KB;  // keys of this block that exist
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < 4; cc++) tmem_ld_32x32b_x32(s_addr + cc * 32, sr[cc]);
      tmem_ld_wait();
      if (valid < KB) {
#pragma unroll
        for (int cc = 0; cc < 4; cc++)
#pragma unroll
          for (int e = 0; e < 32; e++)
            if (cc * 32 + e >= valid) sr[cc][e] = 0xFF800000u;  // -inf
      }
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        mx0 = max3(mx0, __uint_as_float(sr[0][e]), __uint_as_float(sr[0][e + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[1][e]), __uint_as_float(sr[1][e + 1]));
        mx2 = max3(mx2, __uint_as_float(sr[2][e]), __uint_as_float(sr[2][e + 1]));
        mx3 = max3(mx3, __uint_as_float(sr[3][e]), __uint_as_float(sr[3][e + 1]));
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
      const float2 c2 = make_float2(c, c), neg_m2 = make_float2(-m2, -m2);
      uint32_t pk[2][32];
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
      for (int cc = 0; cc < 4; cc++) {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float2 x = ffma2(make_float2(__uint_as_float(sr[cc][e]), __uint_as_float(sr[cc][e + 1])), c2, neg_m2);
          float2 pr;
          pr.x = ex2_approx(x.x);
          pr.y = ex2_approx(x.y);
          if (valid < KB) {  // keys past the end contribute nothing
            if (cc * 32 + e >= valid) pr.x = 0.0f;
            if (cc * 32 + e + 1 >= valid) pr.y = 0.0f;
          }
          if ((e & 2) == 0) la = fadd2(la, pr);
          else lb = fadd2(lb, pr);
          pk[cc >> 1][(cc & 1) * 16 + (e >> 1)] = pack_f16x2(pr.x, pr.y);
        }
      }
      l += (la.x + la.y) + (lb.x + lb.y);
      tmem_st_32x32b_x32(s_addr, pk[0]);
      tmem_st_32x32b_x32(s_addr + 32, pk[1]);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i]);
    }

    if (ok && PH_WARP_WAIT(&o_done[i], 0, SITE_FLASH_EPI, wctx)) {
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
  if (clock_cta) launch_clock_end(clock_slot, p.status);
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
  if (D == 128) {
    e = out_f32 ? launch_d<128, true>(tmQ, tmK, tmV, p, batch_heads, stream)
                : launch_d<128, false>(tmQ, tmK, tmV, p, batch_heads, stream);
  } else {
    e = out_f32 ? launch_d<64, true>(tmQ, tmK, tmV, p, batch_heads, stream)
                : launch_d<64, false>(tmQ, tmK, tmV, p, batch_heads, stream);
  }
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
