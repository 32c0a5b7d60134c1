// Pipe-rate probe for sm_100a: how fast one SM retires tcgen05.mma instructions
// of the shapes the leaf kernels use, and how fast it retires fp32 fmas from
// registers.  The numbers it prints are the per-instruction costs that bound the
// GEMM and flash-attention kernels (see the kernel headers).  Diagnostic only:
// nothing in the library depends on it.
//
//   build:  python phobos-lang_b200/build.py --probes      (writes phobos-lang_b200/pipe_probe)
//   run:    ./phobos-lang_b200/pipe_probe
#include <cstdio>
#include <cuda_runtime.h>

#include "../common.cuh"
using namespace ph;

// ---- tcgen05.mma: `nissue` warps each issue a stream of 128 x N x 16 MMAs into their own accumulator
__global__ void __launch_bounds__(128, 1) umma_rate(int ts_mode, int N, int b_mn, int nissue, int nacc, int whole_warp, int iters, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  __shared__ long long tstart;
  for (int i = threadIdx.x; i < 192 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;  // f16 ones
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; i++) mbar_init(&bar[i], 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc(&slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = slot;
  const int w = threadIdx.x >> 5;
  if (threadIdx.x == 0) tstart = clock64();
  __syncthreads();
  __shared__ volatile int stop_flag;
  if (threadIdx.x == 0) stop_flag = 0;
  __syncthreads();
  if (whole_warp == 4 && w >= nissue) {
    // the other warps keep their schedulers busy with dependent FMAs until the issuer is done
    float v = static_cast<float>(threadIdx.x);
    while (stop_flag == 0) {
#pragma unroll
      for (int i = 0; i < 64; i++) v = fmaf(v, 1.0001f, 0.5f);
    }
    if (v == 12345.678f) out[7] = 1;
  }
  if ((whole_warp == 0 || whole_warp == 3 || whole_warp == 4) && (threadIdx.x & 31) == 0 && w < nissue) {
    const int same = whole_warp == 3 ? 0 : 1;   // 0: every MMA reuses the first k-step's descriptors
    const uint32_t idesc = umma_idesc_f16(128, N, true, false, b_mn != 0);
    const uint32_t a = smem_u32(smem + w * 49152), b = smem_u32(smem + w * 49152 + 16384);
    const uint64_t ad0 = umma_smem_desc(a, 16, 1024);
    const uint64_t bd0 = b_mn ? umma_smem_desc(b, 8192, 1024) : umma_smem_desc(b, 16, 1024);
    const uint64_t bstep = b_mn ? (2048 >> 4) : (32 >> 4);
    const uint32_t d = tb + w * N;
    const uint32_t a_tmem = tb + 256 + (w & 1) * 64;  // TMEM-A runs keep accumulators below column 256
#pragma unroll 1
    for (int it = 0; it < iters; it++) {
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        // with nacc > 1 this one thread rotates over nacc independent accumulators
        const uint32_t dk = d + static_cast<uint32_t>((kk & (nacc - 1)) * N);  // nacc is a power of two
        if (ts_mode) umma_f16_ts(dk, a_tmem + kk * 8 * same, bd0 + kk * bstep * same, idesc, 1);
        else umma_f16_ss(dk, ad0 + kk * 2 * same, bd0 + kk * bstep * same, idesc, 1);
      }
    }
    out[4 + w] = clock64() - tstart;  // the issue loop alone, before the MMAs are known complete
    umma_commit(&bar[w]);
    unsigned spins = 0;
    while (!mbar_try_wait(&bar[w], 0) && ++spins < (1u << 26)) {
    }
    out[w] = clock64() - tstart;
    stop_flag = 1;
  }
  if ((whole_warp == 1 || whole_warp == 2) && w < nissue) {
    const int same = whole_warp == 2 ? 0 : 1;
    // every lane runs the loop and the descriptor arithmetic (warp-uniform values);
    // only the tcgen05.mma itself is predicated on one elected lane
    const uint32_t idesc = umma_idesc_f16(128, N, true, false, b_mn != 0);
    const uint32_t a = smem_u32(smem + w * 49152), b = smem_u32(smem + w * 49152 + 16384);
    const uint64_t ad0 = umma_smem_desc(a, 16, 1024);
    const uint64_t bd0 = b_mn ? umma_smem_desc(b, 8192, 1024) : umma_smem_desc(b, 16, 1024);
    const uint64_t bstep = b_mn ? (2048 >> 4) : (32 >> 4);
    const uint32_t d = tb + w * N;
    const uint32_t a_tmem = tb + 256 + (w & 1) * 64;
#pragma unroll 1
    for (int it = 0; it < iters; it++) {
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        if (elect_one()) {
          if (ts_mode) umma_f16_ts(d, a_tmem + kk * 8 * same, bd0 + kk * bstep * same, idesc, 1);
          else umma_f16_ss(d, ad0 + kk * 2 * same, bd0 + kk * bstep * same, idesc, 1);
        }
      }
    }
    if (elect_one()) {
      out[4 + w] = clock64() - tstart;
      umma_commit(&bar[w]);
      unsigned spins = 0;
      while (!mbar_try_wait(&bar[w], 0) && ++spins < (1u << 26)) {
      }
      out[w] = clock64() - tstart;
    }
    __syncwarp();
  }
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tb, 512);
}

// ---- fp32 fma from registers: 8 x 8 outer product per thread, packed (f32x2) or scalar
__device__ __forceinline__ void ffma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
  asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
template <int PACKED>
__global__ void __launch_bounds__(256, 2) ffma_rate(float* out, int iters, float x) {
  if (PACKED) {
    unsigned long long acc[32], a[8], b[4];
    for (int i = 0; i < 32; i++) acc[i] = 0;
    for (int i = 0; i < 8; i++) {
      float v = x + i + threadIdx.x;
      asm("mov.b64 %0, {%1,%1};" : "=l"(a[i]) : "f"(v));
    }
    for (int i = 0; i < 4; i++) {
      float v = x * i + 1;
      asm("mov.b64 %0, {%1,%1};" : "=l"(b[i]) : "f"(v));
    }
    for (int it = 0; it < iters; it++) {
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) ffma2(acc[i * 4 + j], a[i], b[j]);
    }
    unsigned long long s = 0;
    for (int i = 0; i < 32; i++) s ^= acc[i];
    if (s == 12345) out[0] = 1;
  } else {
    float acc[64], a[8], b[8];
    for (int i = 0; i < 64; i++) acc[i] = 0;
    for (int i = 0; i < 8; i++) {
      a[i] = x + i + threadIdx.x;
      b[i] = x * i + 1;
    }
    for (int it = 0; it < iters; it++) {
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(acc[i * 8 + j]) : "f"(a[i]), "f"(b[j]));
    }
    float s = 0;
    for (int i = 0; i < 64; i++) s += acc[i];
    if (s == 12345.f) out[0] = 1;
  }
}

int main() {
  long long* d;
  cudaMalloc(&d, 64);
  cudaFuncSetAttribute(umma_rate, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  printf("tcgen05.mma kind::f16, M=128, K=16, f32 accumulate; clocks per MMA (ideal N/2)\n");
  const int cfgs[][3] = {{0, 64, 0}, {0, 128, 0}, {0, 128, 1}, {0, 192, 0}, {0, 256, 0}, {0, 256, 1}, {1, 64, 1}, {1, 128, 1}, {1, 256, 1}};
  for (auto& c : cfgs)
    for (int ni : {1, 2, 4}) {
      if (ni * c[1] > 512 || (c[0] && ni * c[1] > 256)) continue;  // accumulators (and the TMEM A operand) must fit 512 columns
      const int iters = 256;
      cudaMemset(d, 0, 64);
      umma_rate<<<148, 128, 200 * 1024>>>(c[0], c[1], c[2], ni, 1, 0, iters, d);
      cudaError_t e = cudaDeviceSynchronize();
      long long h[4];
      cudaMemcpy(h, d, 32, cudaMemcpyDeviceToHost);
      long long mx = 0;
      for (int i = 0; i < ni; i++) mx = h[i] > mx ? h[i] : mx;
      printf("  A from %s, B %s-major, N=%3d, %d issuer(s): %6.1f clk/MMA overall  (ideal %3d)%s\n", c[0] ? "TMEM" : "smem",
             c[2] ? "N" : "K", c[1], ni, static_cast<double>(mx) / (iters * 4 * ni), c[1] / 2,
             e == cudaSuccess ? "" : "  CUDA ERROR");
    }
  printf("one issuing thread rotating over several accumulators (A from smem unless noted)\n");
  const int rot[][3] = {{0, 128, 1}, {0, 256, 1}, {0, 64, 2}, {0, 64, 4}, {0, 128, 2}, {0, 128, 4}, {0, 256, 2}, {1, 64, 2}, {1, 64, 4}, {1, 128, 2}};
  for (auto& c : rot) {
    const int iters = 256;
    cudaMemset(d, 0, 64);
    umma_rate<<<148, 128, 200 * 1024>>>(c[0], c[1], 1, 1, c[2], 0, iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[8];
    cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
    printf("  A from %s, N=%3d, 1 issuer, %d accumulators: %6.1f clk/MMA complete, %6.1f clk/MMA to issue  (ideal %3d)%s\n",
           c[0] ? "TMEM" : "smem", c[1], c[2], static_cast<double>(h[0]) / (iters * 4), static_cast<double>(h[4]) / (iters * 4),
           c[1] / 2, e == cudaSuccess ? "" : "  CUDA ERROR");
  }
  printf("whole warp runs the issue loop, one elected lane issues each MMA\n");
  const int ww[][3] = {{0, 64, 1}, {0, 128, 1}, {0, 128, 2}, {0, 256, 1}, {0, 256, 2}, {1, 64, 1}, {1, 128, 1}, {1, 128, 2}, {1, 256, 1}};
  for (auto& c : ww) {
    const int iters = 256;
    cudaMemset(d, 0, 64);
    umma_rate<<<148, 128, 200 * 1024>>>(c[0], c[1], 1, c[2], 1, 1, iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[8];
    cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
    long long mx = h[0] > h[1] ? h[0] : h[1];
    printf("  A from %s, N=%3d, %d issuer(s): %6.1f clk/MMA complete, %6.1f clk/MMA to issue  (ideal %3d)%s\n",
           c[0] ? "TMEM" : "smem", c[1], c[2], static_cast<double>(mx) / (iters * 4 * c[2]),
           static_cast<double>(h[4]) / (iters * 4), c[1] / 2, e == cudaSuccess ? "" : "  CUDA ERROR");
  }
  printf("every MMA with the same descriptors (no descriptor change between MMAs)\n");
  const int sd[][3] = {{0, 128, 2}, {0, 128, 3}, {1, 128, 2}, {1, 128, 3}, {0, 64, 2}, {0, 256, 2}};
  for (auto& c : sd) {
    const int iters = 256;
    cudaMemset(d, 0, 64);
    umma_rate<<<148, 128, 200 * 1024>>>(c[0], c[1], 1, 1, 1, c[2], iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[8];
    cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
    printf("  A from %s, N=%3d, %s: %6.1f clk/MMA complete, %6.1f clk/MMA to issue  (ideal %3d)%s\n", c[0] ? "TMEM" : "smem",
           c[1], c[2] == 2 ? "whole warp" : "one lane  ", static_cast<double>(h[0]) / (iters * 4),
           static_cast<double>(h[4]) / (iters * 4), c[1] / 2, e == cudaSuccess ? "" : "  CUDA ERROR");
  }
  printf("one issuing lane while the CTA's other three warps run dependent FMAs\n");
  const int bz[][2] = {{0, 64}, {0, 128}, {0, 256}, {1, 128}, {1, 256}};
  for (auto& c : bz) {
    const int iters = 256;
    cudaMemset(d, 0, 64);
    umma_rate<<<148, 128, 200 * 1024>>>(c[0], c[1], 1, 1, 1, 4, iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[8];
    cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
    printf("  A from %s, N=%3d: %6.1f clk/MMA complete  (ideal %3d)%s\n", c[0] ? "TMEM" : "smem", c[1],
           static_cast<double>(h[0]) / (iters * 4), c[1] / 2, e == cudaSuccess ? "" : "  CUDA ERROR");
  }
  float* f;
  cudaMalloc(&f, 4);
  printf("fp32 fma from registers, 256 threads x 2 CTAs per SM\n");
  for (int packed = 1; packed >= 0; packed--) {
    const int iters = 20000, blocks = 296;
    float ms = 0;
    for (int rep = 0; rep < 2; rep++) {
      cudaEvent_t s, t;
      cudaEventCreate(&s);
      cudaEventCreate(&t);
      cudaEventRecord(s);
      if (packed) ffma_rate<1><<<blocks, 256>>>(f, iters, 1.0f);
      else ffma_rate<0><<<blocks, 256>>>(f, iters, 1.0f);
      cudaEventRecord(t);
      cudaEventSynchronize(t);
      cudaEventElapsedTime(&ms, s, t);
    }
    printf("  %s: %.1f TFLOP/s\n", packed ? "fma.rn.f32x2" : "fma.rn.f32  ", 2.0 * 64 * iters * 256.0 * blocks / ms / 1e9);
  }
  return 0;
}
