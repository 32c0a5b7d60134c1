// extern "C" entry points of the leaf executor: argument validation, kernel
// selection by entry name and element types, per-device state.  See
// include/phobos_leaf.h for the contract of every function.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/phobos_leaf.h"
#include "host.h"
#include "kernels.h"

namespace ph {

// ---- last error (thread local) ------------------------------------------------
static thread_local char t_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { t_err[0] = 0; }
const char* last_error() { return t_err; }

// ---- per-device state -----------------------------------------------------------
// Diagnostic block of the device, in the module's device data segment; its address
// is looked up once per device.  Word 0 is written by kernels whose bounded wait
// gave up; words 2..5 hold the launch clock (two 64-bit values, see common.cuh).
__device__ __align__(16) uint32_t g_status_word[8];

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  uint32_t* status = nullptr;
};
static DeviceState g_dev[64];
static std::mutex g_dev_mu;

int device_state(DeviceState** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(PH_ERR_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> g(g_dev_mu);
  DeviceState& s = g_dev[dev];
  if (!s.ready) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
      return fail(PH_ERR_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only (no fallback)", dev,
                  prop.major, prop.minor);
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_status_word);
    if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    e = cudaMemset(p, 0, 8 * sizeof(uint32_t));
    if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "cudaMemset: %s", cudaGetErrorString(e));
    s.sm_count = prop.multiProcessorCount;
    s.cc_major = prop.major;
    s.status = static_cast<uint32_t*>(p);
    s.ready = true;
  }
  *out = &s;
  return PH_OK;
}

// ---- tensor validation ------------------------------------------------------------
struct View {
  char* base;  // ptr + offset, in bytes
  long long rows, cols, ld;
  int dtype;
};

static int view_of(const PhTensor* t, const char* name, View* v) {
  if (!t) return fail(PH_ERR_INVALID, "%s: null tensor descriptor", name);
  if (!t->ptr) return fail(PH_ERR_INVALID, "%s: null data pointer", name);
  if (t->rank != 2) return fail(PH_ERR_INVALID, "%s: rank %d, expected 2", name, t->rank);
  if (t->dtype != PH_F16 && t->dtype != PH_F32)
    return fail(PH_ERR_UNSUPPORTED, "%s: element type %d is not f16 or f32", name, t->dtype);
  const long long es = t->dtype == PH_F16 ? 2 : 4;
  if (t->sizes[0] <= 0 || t->sizes[1] <= 0)
    return fail(PH_ERR_INVALID, "%s: empty extent %lldx%lld", name, (long long)t->sizes[0], (long long)t->sizes[1]);
  if (t->sizes[0] > 0x7fffffffLL || t->sizes[1] > 0x7fffffffLL)
    return fail(PH_ERR_INVALID, "%s: extent exceeds 2^31-1", name);
  if (t->strides[1] != 1) return fail(PH_ERR_INVALID, "%s: inner stride %lld, expected 1", name, (long long)t->strides[1]);
  if (t->strides[0] < t->sizes[1])
    return fail(PH_ERR_INVALID, "%s: row stride %lld smaller than row length %lld", name, (long long)t->strides[0],
                (long long)t->sizes[1]);
  if ((t->strides[0] * es) % 16 != 0)
    return fail(PH_ERR_INVALID, "%s: row stride %lld elements is not a multiple of 16 bytes", name,
                (long long)t->strides[0]);
  if ((t->sizes[1] * es) % 16 != 0)
    return fail(PH_ERR_INVALID, "%s: row length %lld elements is not a multiple of 16 bytes", name,
                (long long)t->sizes[1]);
  if (t->offset < 0) return fail(PH_ERR_INVALID, "%s: negative offset", name);
  char* base = static_cast<char*>(t->ptr) + t->offset * es;
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    return fail(PH_ERR_INVALID, "%s: data pointer is not 16-byte aligned", name);
  v->base = base;
  v->rows = t->sizes[0];
  v->cols = t->sizes[1];
  v->ld = t->strides[0];
  v->dtype = t->dtype;
  return PH_OK;
}

static int map_launch_rc(int rc, const char* what, const char* err) {
  if (rc == 0) return PH_OK;
  if (rc == -2) return fail(PH_ERR_UNSUPPORTED, "%s: %s", what, err);
  if (rc == -1) return fail(PH_ERR_INVALID, "%s: %s", what, err);
  return fail(PH_ERR_DEVICE, "%s: %s", what, err);
}

static size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Tensor-core GEMM dispatch: CTA pairs once the problem spans at least a quarter of a round of
// 256 x 256 pair tiles, the 1-CTA kernel below that.
static bool tc_uses_pairs(long long M, long long N, int sm_count) {
  return ((M + 255) / 256) * ((N + 255) / 256) >= sm_count / 4 && M >= 256 && N >= 128;
}

static int launch_tc(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                     int K, float alpha, float beta, bool acc_f16, bool c_f16, int sm_count, void* workspace,
                     size_t workspace_bytes, uint32_t* status, cudaStream_t stream, const char** err) {
  if (tc_uses_pairs(M, N, sm_count))
    return launch_gemm_tc_pair(A, lda, B, ldb, C, ldc, M, N, K, alpha, beta, acc_f16, c_f16, sm_count, workspace,
                               workspace_bytes, status, stream, err);
  return launch_gemm_tc(A, lda, B, ldb, C, ldc, M, N, K, alpha, beta, acc_f16, c_f16, sm_count, status, stream, err);
}

// Bytes of the rounded f16 copies of f32-stored A [M,K] and B [K,N].
size_t gemm_staging_bytes(long long M, long long N, long long K) {
  return align256(static_cast<size_t>(M) * K * 2) + align256(static_cast<size_t>(K) * N * 2);
}

// SM count of the current device if one is usable, else that of a B200.
static int sm_count_or_default() {
  DeviceState* ds;
  if (device_state(&ds) == PH_OK) return ds->sm_count;
  clear_error();
  return 148;
}

}  // namespace ph

using namespace ph;

extern "C" {

const char* phobos_last_error(void) { return last_error(); }
const char* phobos_version(void) { return "phobos-b200-leaf 0.1 (sm_100a)"; }

size_t phobos_dtype_bytes(int32_t dtype) {
  switch (dtype) {
    case PH_I8: case PH_BOOL: return 1;
    case PH_F16: return 2;
    case PH_F32: case PH_I32: return 4;
    case PH_F64: case PH_I64: return 8;
    default: return 0;
  }
}

int phobos_device_info(int device, PhDeviceInfo* out) {
  clear_error();
  if (!out) return fail(PH_ERR_INVALID, "null output");
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "cudaGetDeviceProperties(%d): %s", device, cudaGetErrorString(e));
  int clock_khz = 0;
  cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, device);
  memset(out, 0, sizeof(*out));
  out->device = device;
  out->sm_count = prop.multiProcessorCount;
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->sm_clock_khz = clock_khz;
  out->total_mem_bytes = static_cast<int64_t>(prop.totalGlobalMem);
  out->fp32_peak_flops = static_cast<double>(prop.multiProcessorCount) * 128.0 * 2.0 * clock_khz * 1e3;
  snprintf(out->name, sizeof(out->name), "%.63s", prop.name);
  return PH_OK;
}

int phobos_device_status(void* stream, uint32_t* status_out) {
  clear_error();
  DeviceState* ds;
  int rc = device_state(&ds);
  if (rc) return rc;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "cudaStreamSynchronize: %s", cudaGetErrorString(e));
  uint32_t w = 0;
  e = cudaMemcpy(&w, ds->status, sizeof(w), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "status read: %s", cudaGetErrorString(e));
  if (w != 0) cudaMemset(ds->status, 0, sizeof(w));
  if (status_out) *status_out = w;
  if (w != 0) return fail(PH_ERR_TIMEOUT, "a device-side wait gave up (site 0x%x, block %u)", w & 0xff, w >> 8);
  return PH_OK;
}

size_t phobos_gemm_workspace_bytes(int32_t kind, int32_t a_dtype, int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return 0;
  size_t bytes = 0;
  if (kind == PH_GEMM_FP32) return gemm_f32_workspace_bytes(M, K);
  if (kind == PH_GEMM_FP16TC_FP32ACC && a_dtype == PH_F32) bytes += gemm_staging_bytes(M, N, K);
  if (kind == PH_GEMM_FP16TC_FP32ACC || kind == PH_GEMM_FP16) {
    const int sms = sm_count_or_default();
    if (tc_uses_pairs(M, N, sms)) bytes += gemm_tc_pair_workspace_bytes((int)M, (int)N, (int)K, sms);
  }
  return bytes;
}

int phobos_gemm(const PhTensor* A, const PhTensor* B, const PhTensor* C, float alpha, float beta, int32_t kind,
                void* workspace, size_t workspace_bytes, void* stream_) {
  clear_error();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  View a, b, c;
  int rc;
  if ((rc = view_of(A, "A", &a)) || (rc = view_of(B, "B", &b)) || (rc = view_of(C, "C", &c))) return rc;
  const long long M = a.rows, K = a.cols, N = b.cols;
  if (b.rows != K) return fail(PH_ERR_INVALID, "A is %lldx%lld but B is %lldx%lld", M, K, b.rows, b.cols);
  if (c.rows != M || c.cols != N) return fail(PH_ERR_INVALID, "C is %lldx%lld, expected %lldx%lld", c.rows, c.cols, M, N);
  DeviceState* ds;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  switch (kind) {
    case PH_GEMM_FP32: {
      if (a.dtype != PH_F32 || b.dtype != PH_F32 || c.dtype != PH_F32)
        return fail(PH_ERR_INVALID, "gemm_fp32 takes f32 A, B and C");
      if (workspace && reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return fail(PH_ERR_WORKSPACE, "workspace is not 256-byte aligned");
      // optional: with room for a transposed copy of A the faster form of the kernel runs
      rc = launch_gemm_f32(reinterpret_cast<const float*>(a.base), a.ld, reinterpret_cast<const float*>(b.base), b.ld,
                           reinterpret_cast<float*>(c.base), c.ld, (int)M, (int)N, (int)K, alpha, beta, workspace,
                           workspace ? workspace_bytes : 0, ds->status, stream, &err);
      return map_launch_rc(rc, "gemm_fp32", err);
    }
    case PH_GEMM_FP16TC_FP32ACC: {
      if (c.dtype != PH_F32) return fail(PH_ERR_INVALID, "gemm_fp16tc_fp32acc takes an f32 C");
      if (a.dtype != b.dtype) return fail(PH_ERR_INVALID, "gemm_fp16tc_fp32acc: A and B element types differ");
      const void* a16 = a.base;
      const void* b16 = b.base;
      long long lda = a.ld, ldb = b.ld;
      char* ws = static_cast<char*>(workspace);
      size_t ws_bytes = workspace ? workspace_bytes : 0;
      if (ws && reinterpret_cast<uintptr_t>(ws) % 256 != 0) return fail(PH_ERR_WORKSPACE, "workspace is not 256-byte aligned");
      if (a.dtype == PH_F32) {
        // the .ph signature: f32 storage, rounded RN-even to f16 when staged
        // (phobos-lang/src/codegen/matmul.rs:2166-2231); here by a convert pass.
        // Everything is validated before the first kernel touches the workspace.
        if ((K * 2) % 16 != 0 || (N * 2) % 16 != 0)
          return fail(PH_ERR_INVALID, "gemm_fp16tc_fp32acc: K and N must be multiples of 8");
        const size_t need = gemm_staging_bytes(M, N, K);
        if (!ws || ws_bytes < need)
          return fail(PH_ERR_WORKSPACE, "gemm_fp16tc_fp32acc with f32 operands needs %zu workspace bytes, got %zu", need,
                      ws_bytes);
        char* wa = ws;
        char* wb = wa + align256(static_cast<size_t>(M) * K * 2);
        if ((rc = launch_f32_to_f16_2d(reinterpret_cast<const float*>(a.base), a.ld, wa, M, K, stream, &err)) ||
            (rc = launch_f32_to_f16_2d(reinterpret_cast<const float*>(b.base), b.ld, wb, K, N, stream, &err)))
          return map_launch_rc(rc, "f32->f16 staging", err);
        a16 = wa;
        b16 = wb;
        lda = K;
        ldb = N;
        ws += need;          // what is left may serve the kernel's own scratch
        ws_bytes -= need;
      }
      rc = launch_tc(a16, lda, b16, ldb, c.base, c.ld, (int)M, (int)N, (int)K, alpha, beta, false, false,
                     ds->sm_count, ws, ws_bytes, ds->status, stream, &err);
      return map_launch_rc(rc, "gemm_fp16tc_fp32acc", err);
    }
    case PH_GEMM_FP16: {
      if (a.dtype != PH_F16 || b.dtype != PH_F16 || c.dtype != PH_F16)
        return fail(PH_ERR_INVALID, "gemm_fp16 takes f16 A, B and C");
      if (workspace && reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return fail(PH_ERR_WORKSPACE, "workspace is not 256-byte aligned");
      rc = launch_tc(a.base, a.ld, b.base, b.ld, c.base, c.ld, (int)M, (int)N, (int)K, alpha, beta, true, true,
                     ds->sm_count, workspace, workspace ? workspace_bytes : 0, ds->status, stream, &err);
      return map_launch_rc(rc, "gemm_fp16", err);
    }
    default:
      return fail(PH_ERR_INVALID, "unknown gemm kind %d", kind);
  }
}

int phobos_matmul_init(const PhTensor* C, float beta, int32_t zero_fill, void* stream) {
  clear_error();
  View c;
  int rc;
  if ((rc = view_of(C, "C", &c))) return rc;
  if (c.dtype != PH_F32) return fail(PH_ERR_UNSUPPORTED, "matmul_init takes an f32 C");
  DeviceState* ds;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_scale_f32(reinterpret_cast<float*>(c.base), c.ld, c.rows, c.cols, beta, zero_fill != 0,
                        static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "matmul_init", err);
}

size_t phobos_flash_workspace_bytes(int32_t dtype, int64_t batch_heads, int64_t Nq, int64_t Nk, int64_t D) {
  if (dtype != PH_F32) return 0;
  return align256(static_cast<size_t>(batch_heads) * Nq * D * 2) + 2 * align256(static_cast<size_t>(batch_heads) * Nk * D * 2);
}

int phobos_flash_attention(const PhTensor* Q, const PhTensor* K, const PhTensor* V, const PhTensor* O, float scale,
                           int64_t batch_heads, void* workspace, size_t workspace_bytes, void* stream_) {
  clear_error();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  View q, k, v, o;
  int rc;
  if ((rc = view_of(Q, "Q", &q)) || (rc = view_of(K, "K", &k)) || (rc = view_of(V, "V", &v)) || (rc = view_of(O, "O", &o)))
    return rc;
  if (batch_heads < 1) return fail(PH_ERR_INVALID, "batch_heads %lld < 1", (long long)batch_heads);
  const long long Nq = q.rows, D = q.cols, Nk = k.rows;
  if (k.cols != D || v.cols != D || o.cols != D || v.rows != Nk || o.rows != Nq)
    return fail(PH_ERR_INVALID, "flash_attention: Q %lldx%lld K %lldx%lld V %lldx%lld O %lldx%lld do not agree", q.rows,
                q.cols, k.rows, k.cols, v.rows, v.cols, o.rows, o.cols);
  if (q.dtype != k.dtype || q.dtype != v.dtype || q.dtype != o.dtype)
    return fail(PH_ERR_INVALID, "flash_attention: Q, K, V, O element types differ");
  if (q.ld != D || k.ld != D || v.ld != D || o.ld != D)
    return fail(PH_ERR_INVALID, "flash_attention: tensors must be contiguous [N, D]");
  if (D != 64 && D != 128) return fail(PH_ERR_UNSUPPORTED, "flash_attention: head dim %lld is not 64 or 128", D);
  DeviceState* ds;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  const void *q16 = q.base, *k16 = k.base, *v16 = v.base;
  if (q.dtype == PH_F32) {
    const size_t need = phobos_flash_workspace_bytes(PH_F32, batch_heads, Nq, Nk, D);
    if (!workspace || workspace_bytes < need)
      return fail(PH_ERR_WORKSPACE, "flash_attention with f32 tensors needs %zu workspace bytes, got %zu", need,
                  workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(PH_ERR_WORKSPACE, "workspace is not 256-byte aligned");
    char* wq = static_cast<char*>(workspace);
    char* wk = wq + align256(static_cast<size_t>(batch_heads) * Nq * D * 2);
    char* wv = wk + align256(static_cast<size_t>(batch_heads) * Nk * D * 2);
    if ((rc = launch_f32_to_f16(reinterpret_cast<const float*>(q.base), wq, (unsigned long long)batch_heads * Nq * D, stream, &err)) ||
        (rc = launch_f32_to_f16(reinterpret_cast<const float*>(k.base), wk, (unsigned long long)batch_heads * Nk * D, stream, &err)) ||
        (rc = launch_f32_to_f16(reinterpret_cast<const float*>(v.base), wv, (unsigned long long)batch_heads * Nk * D, stream, &err)))
      return map_launch_rc(rc, "f32->f16 staging", err);
    q16 = wq;
    k16 = wk;
    v16 = wv;
  }
  rc = launch_flash_f16(q16, k16, v16, o.base, q.dtype == PH_F32 ? 1 : 0, batch_heads, (int)Nq, (int)Nk, (int)D, scale,
                        ds->sm_count, ds->status, stream, &err);
  return map_launch_rc(rc, "flash_attention", err);
}

int phobos_last_launch_clock(void* stream, uint64_t* sm_cycles, uint64_t* timer_ns) {
  clear_error();
  DeviceState* ds;
  int rc = device_state(&ds);
  if (rc) return rc;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "cudaStreamSynchronize: %s", cudaGetErrorString(e));
  unsigned long long w[2] = {0, 0};
  e = cudaMemcpy(w, ds->status + 2, sizeof(w), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(PH_ERR_DEVICE, "launch clock read: %s", cudaGetErrorString(e));
  if (sm_cycles) *sm_cycles = w[0];
  if (timer_ns) *timer_ns = w[1];
  return PH_OK;
}

int phobos_selftest_bounded_wait(uint64_t limit_ns, void* stream) {
  clear_error();
  if (limit_ns == 0 || limit_ns > 1000000000ull)
    return fail(PH_ERR_INVALID, "selftest wait limit %llu ns is not in (0, 1 s]", (unsigned long long)limit_ns);
  DeviceState* ds;
  int rc = device_state(&ds);
  if (rc) return rc;
  const char* err = "";
  rc = launch_selftest_wait(limit_ns, ds->status, static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "selftest_bounded_wait", err);
}

// ---- launch by entry name ---------------------------------------------------------------
// A rank-1 f32 vector view (saxpy): contiguous, 16-byte aligned.
static int vector_of(const PhTensor* t, const char* name, float** base, long long* n) {
  if (!t) return fail(PH_ERR_INVALID, "%s: null tensor descriptor", name);
  if (!t->ptr) return fail(PH_ERR_INVALID, "%s: null data pointer", name);
  if (t->rank != 1) return fail(PH_ERR_INVALID, "%s: rank %d, expected 1", name, t->rank);
  if (t->dtype != PH_F32) return fail(PH_ERR_UNSUPPORTED, "%s: element type %d is not f32", name, t->dtype);
  if (t->sizes[0] <= 0) return fail(PH_ERR_INVALID, "%s: empty extent", name);
  if (t->strides[0] != 1) return fail(PH_ERR_INVALID, "%s: stride %lld, expected 1", name, (long long)t->strides[0]);
  if (t->offset < 0) return fail(PH_ERR_INVALID, "%s: negative offset", name);
  float* b = static_cast<float*>(t->ptr) + t->offset;
  if (reinterpret_cast<uintptr_t>(b) % 16 != 0) return fail(PH_ERR_INVALID, "%s: data pointer is not 16-byte aligned", name);
  *base = b;
  *n = t->sizes[0];
  return PH_OK;
}

int phobos_saxpy(const PhTensor* x, const PhTensor* y, const PhTensor* out, float alpha, void* stream) {
  clear_error();
  float *xp, *yp, *op;
  long long nx, ny, no;
  int rc;
  if ((rc = vector_of(x, "x", &xp, &nx)) || (rc = vector_of(y, "y", &yp, &ny)) || (rc = vector_of(out, "out", &op, &no)))
    return rc;
  if (nx != ny || nx != no) return fail(PH_ERR_INVALID, "saxpy: extents differ (%lld, %lld, %lld)", nx, ny, no);
  DeviceState* ds;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_saxpy(xp, yp, op, static_cast<unsigned long long>(nx), alpha, ds->sm_count, static_cast<cudaStream_t>(stream),
                    &err);
  return map_launch_rc(rc, "saxpy", err);
}

int phobos_kda(const PhTensor* Q, const PhTensor* K, const PhTensor* V, const PhTensor* G, const PhTensor* O, float scale,
               void* stream) {
  clear_error();
  View q, k, v, o;
  int rc;
  if ((rc = view_of(Q, "Q", &q)) || (rc = view_of(K, "K", &k)) || (rc = view_of(V, "V", &v)) || (rc = view_of(O, "O", &o)))
    return rc;
  if (q.dtype != PH_F32 || k.dtype != PH_F32 || v.dtype != PH_F32 || o.dtype != PH_F32)
    return fail(PH_ERR_UNSUPPORTED, "kda takes f32 tensors");
  // G is [N, 1]: a column, so the row-length checks of the matrix views do not apply
  if (!G || !G->ptr) return fail(PH_ERR_INVALID, "G: null tensor");
  if (G->rank != 2 || G->dtype != PH_F32 || G->sizes[1] != 1 || G->strides[0] < 1 || G->offset < 0)
    return fail(PH_ERR_INVALID, "G: expected an f32 [N, 1] tensor");
  const long long N = q.rows, D = q.cols;
  if (k.rows != N || v.rows != N || o.rows != N || G->sizes[0] != N || k.cols != D || v.cols != D || o.cols != D)
    return fail(PH_ERR_INVALID, "kda: Q, K, V, O must be [N, D] and G [N, 1] with the same N and D");
  DeviceState* ds;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_kda(reinterpret_cast<const float*>(q.base), q.ld, reinterpret_cast<const float*>(k.base), k.ld,
                  reinterpret_cast<const float*>(v.base), v.ld, static_cast<const float*>(G->ptr) + G->offset, G->strides[0],
                  reinterpret_cast<float*>(o.base), o.ld, static_cast<int>(N), static_cast<int>(D), scale,
                  static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "kda", err);
}

// kind_hint: -1, or a PhGemmKind / PH_KIND_AUTO in the low byte, optionally | PH_LAUNCH_STEP_LEAF
static bool hint_is_step(int32_t kind_hint) { return kind_hint >= 0 && (kind_hint & PH_LAUNCH_STEP_LEAF) != 0; }
static int gemm_kind_from_types(const PhTensor* t, int32_t kind_hint) {
  const int base = kind_hint < 0 ? -1 : (kind_hint & 0xFF);
  if (base >= 0 && base != PH_KIND_AUTO) return base;
  if (t[0].dtype == PH_F16 && t[2].dtype == PH_F16) return PH_GEMM_FP16;
  if (t[0].dtype == PH_F16 && t[2].dtype == PH_F32) return PH_GEMM_FP16TC_FP32ACC;
  return PH_GEMM_FP32;
}

static int scalar_f32(const PhScalar* s, int32_t n, uint32_t pos, float* out) {
  for (int32_t i = 0; i < n; i++) {
    if (s[i].pos != pos) continue;
    if (s[i].dtype == PH_F32) {
      uint32_t b = static_cast<uint32_t>(s[i].bits);
      memcpy(out, &b, 4);
      return PH_OK;
    }
    if (s[i].dtype == PH_F64) {
      double d;
      memcpy(&d, &s[i].bits, 8);
      *out = static_cast<float>(d);
      return PH_OK;
    }
    return fail(PH_ERR_INVALID, "scalar at position %u has type %d, expected f32", pos, s[i].dtype);
  }
  return fail(PH_ERR_INVALID, "missing scalar at parameter position %u", pos);
}

size_t phobos_launch_workspace_bytes(const char* entry, const PhTensor* t, int32_t n, int32_t kind_hint) {
  if (!entry || !t) return 0;
  if ((!strcmp(entry, "gemm") || !strcmp(entry, "matmul")) && n == 3)
    return phobos_gemm_workspace_bytes(gemm_kind_from_types(t, kind_hint), t[0].dtype, t[0].sizes[0], t[1].sizes[1],
                                       t[0].sizes[1]);
  if (!strcmp(entry, "flash_attention") && n == 4)
    return phobos_flash_workspace_bytes(t[0].dtype, 1, t[0].sizes[0], t[1].sizes[0], t[0].sizes[1]);
  return 0;
}

int phobos_launch(const char* entry, const PhTensor* t, int32_t n_tensors, const PhScalar* scalars, int32_t n_scalars,
                  const uint32_t grid[3], const uint32_t cta[3], int32_t kind_hint, void* workspace,
                  size_t workspace_bytes, void* stream) {
  clear_error();
  if (!entry) return fail(PH_ERR_INVALID, "null entry name");
  if (!grid || !cta) return fail(PH_ERR_INVALID, "%s: COMPUTE needs grid and cta", entry);
  if (grid[0] == 0 || grid[1] == 0 || grid[2] == 0 || cta[0] == 0 || cta[1] == 0 || cta[2] == 0)
    return fail(PH_ERR_INVALID, "%s: empty grid or cta", entry);
  if (n_tensors > 0 && !t) return fail(PH_ERR_INVALID, "%s: null tensor list", entry);
  if (n_scalars > 0 && !scalars) return fail(PH_ERR_INVALID, "%s: null scalar list", entry);
  int rc;
  if (!strcmp(entry, "gemm") || !strcmp(entry, "matmul")) {
    // gemm(A, B, C, alpha, beta): tensors at positions 0..2, scalars at 3 and 4
    if (n_tensors != 3) return fail(PH_ERR_INVALID, "%s takes 3 tensors, got %d", entry, n_tensors);
    float alpha = 1.0f, beta = 1.0f;
    if (hint_is_step(kind_hint)) {
      // The accumulate step of a cluster chain (rewrite_step_store, phobos-cluster/src/
      // clustergen.rs:1363-1399): C = alpha*(A@B) + C.  The COMPUTE still carries the
      // kernel's own scalar list, but the leaf no longer uses beta (the init leaf applied
      // it once); a kernel without an alpha parameter accumulates acc itself.
      bool have_alpha = false;
      for (int32_t i = 0; i < n_scalars; i++) have_alpha = have_alpha || scalars[i].pos == 3;
      if (have_alpha && (rc = scalar_f32(scalars, n_scalars, 3, &alpha))) return rc;
    } else {
      if ((rc = scalar_f32(scalars, n_scalars, 3, &alpha)) || (rc = scalar_f32(scalars, n_scalars, 4, &beta))) return rc;
    }
    return phobos_gemm(&t[0], &t[1], &t[2], alpha, beta, gemm_kind_from_types(t, kind_hint), workspace, workspace_bytes,
                       stream);
  }
  if (!strcmp(entry, "gemm_init") || !strcmp(entry, "matmul_init")) {
    // <kernel>_init(C [, beta]): beta*C when a beta scalar is bound, zero fill otherwise
    if (n_tensors != 1) return fail(PH_ERR_INVALID, "%s takes 1 tensor, got %d", entry, n_tensors);
    if (n_scalars == 0) return phobos_matmul_init(&t[0], 0.0f, 1, stream);
    float beta;
    uint32_t b = static_cast<uint32_t>(scalars[0].bits);
    if (scalars[0].dtype != PH_F32) return fail(PH_ERR_INVALID, "%s: beta must be f32", entry);
    memcpy(&beta, &b, 4);
    return phobos_matmul_init(&t[0], beta, 0, stream);
  }
  if (!strcmp(entry, "flash_attention")) {
    if (n_tensors != 4) return fail(PH_ERR_INVALID, "flash_attention takes 4 tensors, got %d", n_tensors);
    float scale;
    if ((rc = scalar_f32(scalars, n_scalars, 4, &scale))) return rc;
    return phobos_flash_attention(&t[0], &t[1], &t[2], &t[3], scale, 1, workspace, workspace_bytes, stream);
  }
  if (!strcmp(entry, "kda")) {
    // kda(Q, K, V, G, O, scale): examples/kda_fp32.ph
    if (n_tensors != 5) return fail(PH_ERR_INVALID, "kda takes 5 tensors, got %d", n_tensors);
    float scale;
    if ((rc = scalar_f32(scalars, n_scalars, 5, &scale))) return rc;
    return phobos_kda(&t[0], &t[1], &t[2], &t[3], &t[4], scale, stream);
  }
  if (!strcmp(entry, "saxpy")) {
    // saxpy(x, y, out, alpha): examples/saxpy_fp32.ph
    if (n_tensors != 3) return fail(PH_ERR_INVALID, "saxpy takes 3 tensors, got %d", n_tensors);
    float alpha;
    if ((rc = scalar_f32(scalars, n_scalars, 3, &alpha))) return rc;
    return phobos_saxpy(&t[0], &t[1], &t[2], alpha, stream);
  }
  return fail(PH_ERR_UNSUPPORTED, "no native kernel for entry '%s'", entry);
}

// ---- generator and conversions ---------------------------------------------------------------
int phobos_fill_random_device(void* out, int32_t dtype, uint64_t n, uint64_t seed, uint64_t first, float scale,
                              int32_t normal, void* stream) {
  clear_error();
  if (!out && n) return fail(PH_ERR_INVALID, "null output");
  if (dtype != PH_F16 && dtype != PH_F32) return fail(PH_ERR_UNSUPPORTED, "fill: element type %d", dtype);
  DeviceState* ds;
  int rc;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_fill_random(out, dtype == PH_F16, n, seed, first, scale, normal, static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "fill_random", err);
}

int phobos_fill_random_block(void* out, int32_t dtype, uint64_t rows, uint64_t cols, uint64_t ld_out, uint64_t seed,
                             uint64_t first, uint64_t stream_pitch, float scale, void* stream) {
  clear_error();
  if (!out && rows * cols) return fail(PH_ERR_INVALID, "null output");
  if (dtype != PH_F16 && dtype != PH_F32) return fail(PH_ERR_UNSUPPORTED, "fill: element type %d", dtype);
  if (ld_out < cols) return fail(PH_ERR_INVALID, "fill: output pitch %llu smaller than %llu columns",
                                 (unsigned long long)ld_out, (unsigned long long)cols);
  DeviceState* ds;
  int rc;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_fill_random_block(out, dtype == PH_F16, rows, cols, ld_out, seed, first, stream_pitch, scale,
                                static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "fill_random_block", err);
}

int phobos_convert_f32_to_f16(const float* in, void* out, uint64_t n, void* stream) {
  clear_error();
  if ((!in || !out) && n) return fail(PH_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(in) % 16 || reinterpret_cast<uintptr_t>(out) % 8)
    return fail(PH_ERR_INVALID, "convert: pointers must be 16-byte (f32) and 8-byte (f16) aligned");
  DeviceState* ds;
  int rc;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_f32_to_f16(in, out, n, static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "convert_f32_to_f16", err);
}

int phobos_convert_f16_to_f32(const void* in, float* out, uint64_t n, void* stream) {
  clear_error();
  if ((!in || !out) && n) return fail(PH_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(in) % 8 || reinterpret_cast<uintptr_t>(out) % 16)
    return fail(PH_ERR_INVALID, "convert: pointers must be 8-byte (f16) and 16-byte (f32) aligned");
  DeviceState* ds;
  int rc;
  if ((rc = device_state(&ds))) return rc;
  const char* err = "";
  rc = launch_f16_to_f32(in, out, n, static_cast<cudaStream_t>(stream), &err);
  return map_launch_rc(rc, "convert_f16_to_f32", err);
}

}  // extern "C"
