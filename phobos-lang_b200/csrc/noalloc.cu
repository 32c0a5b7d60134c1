// phobos_gemm_fp16tc_noalloc: the f32-storage tensor-core GEMM for callers that
// cannot hand over a workspace.
//
// The `gemm_fp16tc_fp32acc` kernel rounds f32-stored A and B to f16 before the
// MMAs and needs scratch memory for the rounded copies.  phobos_gemm takes that
// scratch from the caller.  Some callers have none to give and must not create
// any: a pod that handed its entire device budget to the tile arena at start-up,
// a serving loop that is forbidden to enter the CUDA allocator once it is
// running, a plugin host that owns all allocation itself.  For them the scratch
// lives in this library's own device data segment: a fixed array that every GPU
// which loads the library carries until the process exits.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/phobos_leaf.h"
#include "host.h"

namespace {

// Rounded copies of A (M*K f16) and B (K*N f16), each padded to 256 bytes.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PH_NOALLOC_SCRATCH_BYTES];

// Device address of the array, looked up once per device.  In host code the
// array's name is only a handle for the runtime; the address a kernel can use
// comes from cudaGetSymbolAddress with that device current.
void* g_scratch_addr[64] = {};
std::mutex g_scratch_mu;

int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ph::fail(PH_ERR_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return ph::fail(PH_ERR_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> g(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return ph::fail(PH_ERR_DEVICE, "cudaGetSymbolAddress(scratch) on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return PH_OK;
}

}  // namespace

extern "C" int phobos_gemm_fp16tc_noalloc(const PhTensor* A, const PhTensor* B, const PhTensor* C, float alpha,
                                          float beta, void* stream) {
  ph::clear_error();
  if (!A || !B || !C) return ph::fail(PH_ERR_INVALID, "null tensor descriptor");
  if (A->dtype != PH_F32 || B->dtype != PH_F32 || C->dtype != PH_F32)
    return ph::fail(PH_ERR_INVALID, "phobos_gemm_fp16tc_noalloc takes f32-stored A, B and C");
  if (A->rank != 2 || B->rank != 2) return ph::fail(PH_ERR_INVALID, "A and B must have rank 2");
  const int64_t M = A->sizes[0], K = A->sizes[1], N = B->sizes[1];
  if (M <= 0 || N <= 0 || K <= 0) return ph::fail(PH_ERR_INVALID, "A is %lldx%lld, B has %lld columns", (long long)M, (long long)K, (long long)N);
  const size_t need = ph::gemm_staging_bytes(M, N, K);
  if (need > static_cast<size_t>(PH_NOALLOC_SCRATCH_BYTES))
    return ph::fail(PH_ERR_WORKSPACE,
                    "phobos_gemm_fp16tc_noalloc: M=%lld N=%lld K=%lld needs %zu scratch bytes, the built-in scratch holds %d "
                    "(2*(M*K + K*N) bytes must fit); use phobos_gemm with a caller workspace for larger problems",
                    (long long)M, (long long)N, (long long)K, need, PH_NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: the convert pass overwrites
  // every byte the GEMM reads before the GEMM runs, on the same stream.
  return phobos_gemm(A, B, C, alpha, beta, PH_GEMM_FP16TC_FP32ACC, scratch, PH_NOALLOC_SCRATCH_BYTES, stream);
}
