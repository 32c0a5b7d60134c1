// HBM-bound helper kernels: the seeded input generator and f32 <-> f16
// conversion passes.
//
// Generator: Lcg of phobos-base/src/rng.rs:9-20,
//   state <- state * 6364136223846793005 + 1442695040888963407 (mod 2^64)
//   unit  =  f32(state >> 33) / 2^31 - 1.0            in [-1, 1)
// which is what `phobos-tensor init --fill random` writes
// (phobos-cluster/src/bin/phobos-tensor.rs:55-72).  Each thread jumps to its
// slice of the stream with the closed form of the affine recurrence and then
// steps sequentially, so the values are those of the sequential generator.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

constexpr unsigned long long LCG_A = 6364136223846793005ull;
constexpr unsigned long long LCG_C = 1442695040888963407ull;
constexpr int PER_THREAD = 64;

__host__ __device__ inline unsigned long long lcg_skip(unsigned long long s, unsigned long long n) {
  unsigned long long a = LCG_A, c = LCG_C, acc_a = 1, acc_c = 0;
  while (n) {
    if (n & 1) {
      acc_a = acc_a * a;
      acc_c = acc_c * a + c;
    }
    c = (a + 1) * c;
    a = a * a;
    n >>= 1;
  }
  return acc_a * s + acc_c;
}

__device__ inline float lcg_unit(unsigned long long& s) {
  s = s * LCG_A + LCG_C;
  return __fsub_rn(__fmul_rn(__ull2float_rn(s >> 33), 4.656612873077393e-10f /* 2^-31 */), 1.0f);
}

template <typename T>
__device__ inline void put(T* out, unsigned long long i, float v);
template <>
__device__ inline void put<float>(float* out, unsigned long long i, float v) {
  out[i] = v;
}
template <>
__device__ inline void put<__half>(__half* out, unsigned long long i, float v) {
  out[i] = __float2half_rn(v);
}

template <typename T>
__global__ void fill_uniform_kernel(T* out, unsigned long long n, unsigned long long seed,
                                    unsigned long long first, float scale) {
  const unsigned long long t = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  const unsigned long long lo = t * PER_THREAD;
  if (lo >= n) return;
  const unsigned long long hi = lo + PER_THREAD < n ? lo + PER_THREAD : n;
  unsigned long long s = lcg_skip(seed, first + lo);
  for (unsigned long long i = lo; i < hi; i++) put<T>(out, i, __fmul_rn(scale, lcg_unit(s)));
}

// Block variant: row r of the output takes stream elements first + r*pitch + [0, cols).
template <typename T>
__global__ void fill_block_kernel(T* out, unsigned long long rows, unsigned long long cols, unsigned long long ld_out,
                                  unsigned long long seed, unsigned long long first, unsigned long long pitch,
                                  float scale) {
  const unsigned long long runs_per_row = (cols + PER_THREAD - 1) / PER_THREAD;
  const unsigned long long t = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  if (t >= rows * runs_per_row) return;
  const unsigned long long r = t / runs_per_row, lo = (t - r * runs_per_row) * PER_THREAD;
  const unsigned long long hi = lo + PER_THREAD < cols ? lo + PER_THREAD : cols;
  unsigned long long s = lcg_skip(seed, first + r * pitch + lo);
  for (unsigned long long c = lo; c < hi; c++) put<T>(out, r * ld_out + c, __fmul_rn(scale, lcg_unit(s)));
}

// N(0,1): Box-Muller over stream pairs (2p, 2p+1): u1 = ((s>>33)+1)/2^31 in
// (0,1], u2 = (s>>33)/2^31 in [0,1).  Element 2p is r cos(2 pi u2), 2p+1 is
// r sin(2 pi u2).  `first` must be even.
template <typename T>
__global__ void fill_normal_kernel(T* out, unsigned long long n, unsigned long long seed,
                                   unsigned long long first, float scale) {
  const unsigned long long t = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  const unsigned long long pairs = (n + 1) / 2;
  const unsigned long long lo = t * (PER_THREAD / 2);
  if (lo >= pairs) return;
  const unsigned long long hi = lo + PER_THREAD / 2 < pairs ? lo + PER_THREAD / 2 : pairs;
  unsigned long long s = lcg_skip(seed, first + 2 * lo);
  for (unsigned long long p = lo; p < hi; p++) {
    s = s * LCG_A + LCG_C;
    const double u1 = (static_cast<double>(s >> 33) + 1.0) / 2147483648.0;
    s = s * LCG_A + LCG_C;
    const double u2 = static_cast<double>(s >> 33) / 2147483648.0;
    const double r = sqrt(-2.0 * log(u1));
    double sn, cs;
    sincos(6.283185307179586476925 * u2, &sn, &cs);
    put<T>(out, 2 * p, __fmul_rn(scale, static_cast<float>(r * cs)));
    if (2 * p + 1 < n) put<T>(out, 2 * p + 1, __fmul_rn(scale, static_cast<float>(r * sn)));
  }
}

__global__ void f32_to_f16_kernel(const float4* __restrict__ in, uint2* __restrict__ out, unsigned long long n4,
                                  const float* in_tail, __half* out_tail, int tail) {
  for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
    const float4 v = in[i];
    __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<unsigned*>(&lo);
    o.y = *reinterpret_cast<unsigned*>(&hi);
    out[i] = o;
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail)
    out_tail[threadIdx.x] = __float2half_rn(in_tail[threadIdx.x]);
}

__global__ void f16_to_f32_kernel(const uint2* __restrict__ in, float4* __restrict__ out, unsigned long long n4,
                                  const __half* in_tail, float* out_tail, int tail) {
  for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
    const uint2 v = in[i];
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    out[i] = make_float4(a.x, a.y, b.x, b.y);
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail)
    out_tail[threadIdx.x] = __half2float(in_tail[threadIdx.x]);
}

// rows x cols (cols % 4 == 0), input pitch ld_in floats, output contiguous f16.
__global__ void f32_to_f16_2d_kernel(const float* __restrict__ in, long long ld_in, uint2* __restrict__ out,
                                     long long rows, long long cols4) {
  const long long total = rows * cols4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols4, c = i - r * cols4;
    const float4 v = *(reinterpret_cast<const float4*>(in + r * ld_in) + c);
    __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<unsigned*>(&lo);
    o.y = *reinterpret_cast<unsigned*>(&hi);
    out[i] = o;
  }
}

// out = alpha * x + y (examples/saxpy_fp32.ph:1-5).  One rounded multiply and one rounded add
// per element, as the reference's own check computes it (verify_saxpy, phobos-bench/src/
// main.rs:1179-1188): results are bit-identical to that, not to a fused multiply-add.
// Pure streaming, 12 bytes of HBM traffic per element.
__device__ __forceinline__ float4 saxpy4(float alpha, float4 a, float4 b) {
  return make_float4(__fadd_rn(__fmul_rn(alpha, a.x), b.x), __fadd_rn(__fmul_rn(alpha, a.y), b.y),
                     __fadd_rn(__fmul_rn(alpha, a.z), b.z), __fadd_rn(__fmul_rn(alpha, a.w), b.w));
}
// One CTA per contiguous run of BLOCK * UNR float4: every thread loads UNR vectors of x and UNR of y
// (streaming, evict-first hints) before its first store, no loop; the hardware block scheduler balances
// the SMs.  Measured 6530 GB/s at 2^25 elements with BLOCK 256, UNR 4 against 5918 GB/s for a
// persistent grid-stride kernel of 4 CTAs per SM (its last wave leaves SMs idle).
template <int BLOCK, int UNR>
__global__ void __launch_bounds__(BLOCK) saxpy_once_kernel(const float4* __restrict__ x, const float4* __restrict__ y,
                                                           float4* __restrict__ out, unsigned long long n4, float alpha,
                                                           const float* x_tail, const float* y_tail, float* out_tail, int tail) {
  const unsigned long long base = static_cast<unsigned long long>(blockIdx.x) * (BLOCK * UNR) + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  float4 a[UNR], b[UNR];
#pragma unroll
  for (int u = 0; u < UNR; u++) {
    const unsigned long long i = base + static_cast<unsigned long long>(u) * BLOCK;
    if (i < n4) {
      a[u] = __ldcs(x + i);
      b[u] = __ldcs(y + i);
    }
  }
#pragma unroll
  for (int u = 0; u < UNR; u++) {
    const unsigned long long i = base + static_cast<unsigned long long>(u) * BLOCK;
    if (i < n4) __stcs(out + i, saxpy4(alpha, a[u], b[u]));
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail)
    out_tail[threadIdx.x] = __fadd_rn(__fmul_rn(alpha, x_tail[threadIdx.x]), y_tail[threadIdx.x]);
}

int grid_for(unsigned long long work_items) {
  unsigned long long b = (work_items + 255) / 256;
  const unsigned long long cap = 148ull * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

int check(const char** err) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace

unsigned long long lcg_skip_host(unsigned long long s, unsigned long long n) { return lcg_skip(s, n); }

int launch_fill_random(void* out, int dtype_is_f16, unsigned long long n, unsigned long long seed,
                       unsigned long long first, float scale, int normal, cudaStream_t stream, const char** err) {
  if (n == 0) return 0;
  const unsigned long long threads = (n + PER_THREAD - 1) / PER_THREAD;
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  if (normal) {
    if (first & 1) {
      *err = "normal fill needs an even stream position";
      return -1;
    }
    if (dtype_is_f16)
      fill_normal_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<__half*>(out), n, seed, first, scale);
    else
      fill_normal_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<float*>(out), n, seed, first, scale);
  } else {
    if (dtype_is_f16)
      fill_uniform_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<__half*>(out), n, seed, first, scale);
    else
      fill_uniform_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<float*>(out), n, seed, first, scale);
  }
  return check(err);
}

int launch_fill_random_block(void* out, int dtype_is_f16, unsigned long long rows, unsigned long long cols,
                             unsigned long long ld_out, unsigned long long seed, unsigned long long first,
                             unsigned long long stream_pitch, float scale, cudaStream_t stream, const char** err) {
  if (rows == 0 || cols == 0) return 0;
  const unsigned long long threads = rows * ((cols + PER_THREAD - 1) / PER_THREAD);
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  if (dtype_is_f16)
    fill_block_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<__half*>(out), rows, cols, ld_out, seed, first,
                                                         stream_pitch, scale);
  else
    fill_block_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<float*>(out), rows, cols, ld_out, seed, first,
                                                        stream_pitch, scale);
  return check(err);
}

int launch_f32_to_f16(const float* in, void* out, unsigned long long n, cudaStream_t stream, const char** err) {
  if (n == 0) return 0;
  const unsigned long long n4 = n / 4;
  const int tail = static_cast<int>(n - n4 * 4);
  f32_to_f16_kernel<<<grid_for(n4), 256, 0, stream>>>(reinterpret_cast<const float4*>(in),
                                                      reinterpret_cast<uint2*>(out), n4, in + n4 * 4,
                                                      static_cast<__half*>(out) + n4 * 4, tail);
  return check(err);
}

int launch_f16_to_f32(const void* in, float* out, unsigned long long n, cudaStream_t stream, const char** err) {
  if (n == 0) return 0;
  const unsigned long long n4 = n / 4;
  const int tail = static_cast<int>(n - n4 * 4);
  f16_to_f32_kernel<<<grid_for(n4), 256, 0, stream>>>(reinterpret_cast<const uint2*>(in),
                                                      reinterpret_cast<float4*>(out), n4,
                                                      static_cast<const __half*>(in) + n4 * 4, out + n4 * 4, tail);
  return check(err);
}

int launch_f32_to_f16_2d(const float* in, long long ld_in, void* out, long long rows, long long cols,
                         cudaStream_t stream, const char** err) {
  if (rows * cols == 0) return 0;
  f32_to_f16_2d_kernel<<<grid_for(rows * (cols / 4)), 256, 0, stream>>>(in, ld_in, reinterpret_cast<uint2*>(out),
                                                                         rows, cols / 4);
  return check(err);
}

int launch_saxpy(const float* x, const float* y, float* out, unsigned long long n, float alpha, int sm_count,
                 cudaStream_t stream, const char** err) {
  if (n == 0) return 0;
  const unsigned long long n4 = n / 4;
  const int tail = static_cast<int>(n - n4 * 4);
  constexpr int BLOCK = 256, UNR = 4;
  (void)sm_count;
  const unsigned long long blocks = (n4 + BLOCK * UNR - 1) / (BLOCK * UNR);
  cudaError_t e = launch_with_pdl(saxpy_once_kernel<BLOCK, UNR>, dim3(static_cast<unsigned>(blocks < 1 ? 1 : blocks)),
                                  dim3(BLOCK), 0, stream, reinterpret_cast<const float4*>(x),
                                  reinterpret_cast<const float4*>(y), reinterpret_cast<float4*>(out), n4, alpha,
                                  static_cast<const float*>(x + n4 * 4), static_cast<const float*>(y + n4 * 4), out + n4 * 4, tail);
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
