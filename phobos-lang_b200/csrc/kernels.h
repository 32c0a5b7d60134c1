// Internal launcher interface between api.cu and the kernel translation units.
#pragma once
#include <cstdlib>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ph {

// Launches `kernel` so that its prologue may overlap the tail of the kernel before it on the stream
// (programmatic stream serialization); the kernel calls pdl_wait() before its first dependent access.
// PHOBOS_PDL=0 falls back to an ordinary launch.
template <typename... KArgs, typename... Args>
cudaError_t launch_with_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  static const bool off = [] {
    const char* e = getenv("PHOBOS_PDL");
    return e && e[0] == '0';
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = off ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}


// gemm_tc.cu — f16 operands on tcgen05 tensor cores.
int launch_gemm_tc(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                   int K, float alpha, float beta, bool acc_f16, bool c_f16, int sm_count,
                   uint32_t* status, cudaStream_t stream, const char** err);
// gemm_tc2.cu — the same operator on CTA pairs (cta_group::2), for large problems.  `workspace` (optional,
// gemm_tc_pair_workspace_bytes, 256-byte aligned) lets the kernel share out its last rounds of tiles by k-blocks.
int launch_gemm_tc_pair(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                        int K, float alpha, float beta, bool acc_f16, bool c_f16, int sm_count, void* workspace,
                        size_t workspace_bytes, uint32_t* status, cudaStream_t stream, const char** err);
size_t gemm_tc_pair_workspace_bytes(int M, int N, int K, int sm_count);

// tmap.cu — TMA descriptors (cuTensorMapEncodeTiled through the runtime's driver entry point).
enum TmapType { TMAP_F16 = 0, TMAP_F32 = 1 };
enum TmapSwizzle { TMAP_SWIZZLE_NONE = 0, TMAP_SWIZZLE_32B = 1, TMAP_SWIZZLE_64B = 2, TMAP_SWIZZLE_128B = 3 };
// Row-major [rows, cols] tensor with row pitch ld_elems; box [box_rows, box_cols].
// tmap_out points at 128 bytes, 64-byte aligned (a CUtensorMap).
bool make_tmap_2d(void* tmap_out, const void* base, TmapType type, long long rows, long long cols,
                  long long ld_elems, int box_rows, int box_cols, TmapSwizzle swizzle);
// [batch, rows, cols] tensor: batch pitch in elements; box [1, box_rows, box_cols].
bool make_tmap_3d(void* tmap_out, const void* base, TmapType type, long long batch, long long rows, long long cols,
                  long long ld_elems, long long batch_pitch_elems, int box_rows, int box_cols, TmapSwizzle swizzle);

// gemm_f32.cu — FFMA GEMM and the matmul_init leaf.  With `workspace` of at least
// gemm_f32_workspace_bytes(M, K) bytes (256-byte aligned) a transposed copy of A is written there first and
// the faster form of the kernel runs; the result is bit-identical either way.
size_t gemm_f32_workspace_bytes(long long M, long long K);
int launch_gemm_f32(const float* A, long long lda, const float* B, long long ldb, float* C, long long ldc, int M,
                    int N, int K, float alpha, float beta, void* workspace, size_t workspace_bytes, uint32_t* status,
                    cudaStream_t stream, const char** err);
int launch_scale_f32(float* C, long long ldc, long long rows, long long cols, float beta, bool zero_fill,
                     cudaStream_t stream, const char** err);

// flash.cu — flash attention forward, f16 operands.
// out_f32 != 0: O is f32 (flash_fp32), otherwise f16.
int launch_flash_f16(const void* Q, const void* K, const void* V, void* O, int out_f32, long long batch_heads,
                     int Nq, int Nk, int D, float scale, int sm_count, uint32_t* status, cudaStream_t stream,
                     const char** err);

// selftest.cu — one CTA whose barrier wait must run out after limit_ns (bounded-wait self-test).
int launch_selftest_wait(unsigned long long limit_ns, uint32_t* status, cudaStream_t stream, const char** err);

// elementwise.cu — generator and conversions.
int launch_fill_random(void* out, int dtype_is_f16, unsigned long long n, unsigned long long seed,
                       unsigned long long first, float scale, int normal, cudaStream_t stream, const char** err);
int launch_fill_random_block(void* out, int dtype_is_f16, unsigned long long rows, unsigned long long cols,
                             unsigned long long ld_out, unsigned long long seed, unsigned long long first,
                             unsigned long long stream_pitch, float scale, cudaStream_t stream, const char** err);
int launch_f32_to_f16(const float* in, void* out, unsigned long long n, cudaStream_t stream, const char** err);
int launch_f16_to_f32(const void* in, float* out, unsigned long long n, cudaStream_t stream, const char** err);
// Chunkwise gated linear attention of one head (examples/kda_fp32.ph): Q, K, V, O [N, D], G [N, 1]; D = 64
int launch_kda(const float* Q, long long ldq, const float* K, long long ldk, const float* V, long long ldv, const float* G,
               long long ldg, float* O, long long ldo, int N, int D, float scale, cudaStream_t stream, const char** err);
// out = alpha * x + y, one rounded multiply and one rounded add per element
int launch_saxpy(const float* x, const float* y, float* out, unsigned long long n, float alpha, int sm_count,
                 cudaStream_t stream, const char** err);
// Strided 2-D f32 -> contiguous f16 (rows x cols), used to stage f32-stored tensor-core operands.
int launch_f32_to_f16_2d(const float* in, long long ld_in, void* out, long long rows, long long cols,
                         cudaStream_t stream, const char** err);

}  // namespace ph
