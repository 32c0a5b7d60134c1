/*
 * phobos_leaf.h — C ABI of the B200 leaf executor for phobos kernels.
 *
 * Every entry point is plain C (pointers, sizes, scalars by value) so that a
 * Rust `extern "C"` block, cgo, JNI or ctypes can bind it unchanged.  Each
 * declaration names the reference interface it stands in for, by file:line in
 * the phobos repository.  All device pointers are CUDA device addresses owned
 * by the caller; unless stated otherwise a call only ENQUEUES work on
 * `stream` (a cudaStream_t passed as void*) and allocates nothing.
 *
 * Return value: 0 on success, a negative PhStatus otherwise; the message of
 * the last failure on the calling thread is returned by phobos_last_error().
 * There is no CPU fallback: without a usable sm_100 device every compute call
 * fails with PH_ERR_DEVICE.
 */
#ifndef PHOBOS_LEAF_H_
#define PHOBOS_LEAF_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define PH_API __attribute__((visibility("default")))
#else
#define PH_API
#endif

/* ---- status codes ------------------------------------------------------ */
typedef enum PhStatus {
  PH_OK = 0,
  PH_ERR_INVALID = -1,    /* bad argument: rank, dtype, stride, alignment, shape mismatch */
  PH_ERR_UNSUPPORTED = -2,/* a combination this executor has no kernel for */
  PH_ERR_DEVICE = -3,     /* CUDA error, or no sm_100 device */
  PH_ERR_WORKSPACE = -4,  /* caller workspace missing or too small */
  PH_ERR_TIMEOUT = -5,    /* a bounded device-side wait gave up (see phobos_device_status) */
  PH_ERR_IO = -6,         /* file:// storage error */
  PH_ERR_PARSE = -7,      /* job file syntax */
  PH_ERR_STATE = -8       /* executor: unknown tile, arena exhausted, dependency cycle */
} PhStatus;

/* ---- element types: order of phobos-cluster/src/tile.rs:33-41 ---------- */
typedef enum PhDataType {
  PH_F16 = 0, PH_F32 = 1, PH_F64 = 2, PH_I8 = 3, PH_I32 = 4, PH_I64 = 5, PH_BOOL = 6
} PhDataType;

/* bytes per element: phobos-cluster/src/tile.rs:43-52 */
PH_API size_t phobos_dtype_bytes(int32_t dtype);

/* ---- tensor descriptor -------------------------------------------------- *
 * Stands in for the "exploded memref" the reference passes per tensor
 * (alloc ptr, aligned ptr, offset, sizes[rank], strides[rank]; i32 or i64
 * fields): phobos-bench/src/main.rs:290-327 and phobos-pod/src/engine.rs:588-601.
 * `ptr` is the aligned pointer; `offset`, `sizes`, `strides` are in elements.
 * Requirements (violations return PH_ERR_INVALID, never undefined behaviour):
 * rank 1 or 2, inner stride 1, (ptr + offset) 16-byte aligned, row stride a
 * multiple of 16 bytes — the reference assumes the same (SPEC.md:62).        */
typedef struct PhTensor {
  void *ptr;
  int32_t dtype; /* PhDataType */
  int32_t rank;
  int64_t sizes[2];
  int64_t strides[2];
  int64_t offset;
} PhTensor;

/* ---- scalar argument ---------------------------------------------------- *
 * phobos-cluster/src/isa.rs:7-11 (ScalarArg{pos,value}) with the value held
 * as the little-endian bit pattern of ScalarValue::to_bits, tile.rs:75-83.   */
typedef struct PhScalar {
  uint32_t pos;   /* parameter position in the kernel signature */
  int32_t dtype;  /* PH_F32, PH_F64, PH_I32, PH_I64, PH_BOOL */
  uint64_t bits;
} PhScalar;

/* ---- which GEMM regime --------------------------------------------------- *
 * The three `gemm` kernels of the reference share one signature and differ in
 * element types and accumulator (examples/gemm_fp32.ph, gemm_fp16tc_fp32acc.ph,
 * gemm_fp16.ph).                                                             */
typedef enum PhGemmKind {
  PH_GEMM_FP32 = 0,           /* f32 A,B,C; FFMA, no TF32            (gemm_fp32.ph:1-22) */
  PH_GEMM_FP16TC_FP32ACC = 1, /* A,B f16 (or f32 rounded RN to f16 on the way in), C f32,
                                 f32 accumulate                      (gemm_fp16tc_fp32acc.ph:1-23) */
  PH_GEMM_FP16 = 2            /* f16 A,B,C, f16 accumulate, f32 epilogue (gemm_fp16.ph:1-23) */
} PhGemmKind;

/* ---- library / device ---------------------------------------------------- */
PH_API const char *phobos_last_error(void);
PH_API const char *phobos_version(void);

typedef struct PhDeviceInfo {
  int32_t device;
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  int32_t sm_clock_khz;       /* cudaDevAttrClockRate */
  int64_t total_mem_bytes;
  double fp32_peak_flops;     /* sm_count * 128 lanes * 2 * clock: the FP32 CUDA-core roofline */
  char name[64];
} PhDeviceInfo;
PH_API int phobos_device_info(int device, PhDeviceInfo *out);

/* Word written by a kernel whose bounded wait gave up (0 = none since the last
 * reset).  Reads and clears the current device's status word; synchronises
 * `stream` first. */
PH_API int phobos_device_status(void *stream, uint32_t *status_out);

/* ---- GEMM: C = alpha * A@B + beta * C ------------------------------------ *
 * Replaces launch_gemm(func, grid, block, stream, a, b, c, M, N, K, alpha,
 * beta, wide) of phobos-bench/src/main.rs:290-327 and the `gemm`/`matmul`
 * COMPUTE of phobos-pod/src/engine.rs:542-653.  A[M,K], B[K,N], C[M,N],
 * row-major.  C is read even when beta == 0 (the reference computes
 * 0*C_old; phobos-lang/src/codegen/matmul.rs:393-402).  Non-blocking.
 * `workspace` (256-byte aligned, phobos_gemm_workspace_bytes bytes) is
 * REQUIRED for PH_GEMM_FP16TC_FP32ACC with f32-stored A/B (the rounded copies)
 * and OPTIONAL otherwise: the tensor-core kinds use it to share their last
 * rounds of tiles between CTA pairs, PH_GEMM_FP32 writes a transposed copy of
 * A there and runs the faster form of its kernel (about 1.1x; without it, or
 * with less than the size asked for, A is read in place).  The result does
 * not depend on it for PH_GEMM_FP32 (bit-identical), and only in the order of
 * two f32 partial sums for the tensor-core kinds.  Calls that share a
 * workspace must not overlap on the GPU.                                      */
PH_API int phobos_gemm(const PhTensor *A, const PhTensor *B, const PhTensor *C, float alpha, float beta,
                       int32_t kind, void *workspace, size_t workspace_bytes, void *stream);
PH_API size_t phobos_gemm_workspace_bytes(int32_t kind, int32_t a_dtype, int64_t M, int64_t N, int64_t K);

/* The same GEMM for callers that have no workspace to lend and may not allocate
 * one (a pod whose whole device budget already went to its tile arena, a
 * serving loop barred from the CUDA allocator, a host that owns all
 * allocation).  It has no counterpart in the reference.  A, B and C are
 * f32-stored (kind PH_GEMM_FP16TC_FP32ACC: A and B are rounded RN-even to f16
 * on the way in); the rounded copies go to a fixed scratch array inside the
 * library's device data, PH_NOALLOC_SCRATCH_BYTES per GPU for as long as the
 * library is loaded.  Limit: 2*(M*K + K*N) bytes (each operand padded to 256)
 * must fit, else PH_ERR_WORKSPACE.  The call allocates nothing and enqueues on
 * `stream` like phobos_gemm.  The first call on a device looks up the scratch
 * address (cudaGetSymbolAddress, with that device current); make that first call
 * before any stream capture begins.  All calls on a device share the one scratch
 * array, which keeps the previous call's bytes (nothing needs to start at zero:
 * each call overwrites what it reads): calls whose kernels may overlap on the
 * GPU (different streams, no ordering) race on it and must be serialised by the
 * caller.                                                                      */
#define PH_NOALLOC_SCRATCH_BYTES (8 << 20)
PH_API int phobos_gemm_fp16tc_noalloc(const PhTensor *A, const PhTensor *B, const PhTensor *C, float alpha,
                                      float beta, void *stream);

/* The init leaf of a partitioned matmul: C = beta * C, or C = 0 when there is
 * no previous value (phobos-cluster/src/clustergen.rs:1276-1360; entry name
 * `<kernel>_init`, clustergen.rs:1288).  The step leaf is phobos_gemm with
 * beta = 1 (clustergen.rs:1363-1399).                                         */
PH_API int phobos_matmul_init(const PhTensor *C, float beta, int32_t zero_fill, void *stream);

/* ---- flash attention ------------------------------------------------------ *
 * Replaces launch_flash(...) of phobos-bench/src/main.rs:334-371 and the
 * `flash_attention` COMPUTE.  Q,O: [Nq,D]; K,V: [Nk,D] row-major
 * (examples/flash_attention_fp16.ph:11-16).  `batch_heads` independent
 * problems are run in one launch; problem h uses the descriptors advanced by
 * h*Nq*D (Q,O) and h*Nk*D (K,V) elements.  Element type f16 (flash_fp16) or
 * f32 (flash_fp32: operands rounded to f16 for the tensor cores as the
 * reference does, phobos-lang/src/codegen/matmul.rs:1592-1597; needs
 * workspace).  D must be 64 or 128.                                          */
PH_API int phobos_flash_attention(const PhTensor *Q, const PhTensor *K, const PhTensor *V, const PhTensor *O,
                                  float scale, int64_t batch_heads, void *workspace, size_t workspace_bytes,
                                  void *stream);
PH_API size_t phobos_flash_workspace_bytes(int32_t dtype, int64_t batch_heads, int64_t Nq, int64_t Nk, int64_t D);

/* Diagnostic (no reference counterpart; the reference derives its fp32 peak from the
 * device's nominal clock, phobos-bench/src/report.rs:125-147): the SM clock a launch
 * actually ran at.  One CTA of every GEMM and flash launch records how many SM cycles
 * and how many nanoseconds of the global timer it lived; this call synchronises
 * `stream` and returns the pair of the most recent such launch on the current device
 * (cycles / ns = GHz).  The timer ticks in steps of up to 1 us, so the ratio is
 * meaningful for launches of tens of microseconds and longer.                      */
PH_API int phobos_last_launch_clock(void *stream, uint64_t *sm_cycles, uint64_t *timer_ns);

/* Self-test of the bounded-wait policy (the analogue of the reference's stall detector
 * and fetch deadline, phobos-pod/src/engine.rs:752-775, 825-828): launches one CTA that
 * waits on a barrier nobody arrives at, with a limit of `limit_ns`.  The kernel gives up
 * when the limit passes, records its site code and ends normally; the next
 * phobos_device_status() call on the device then reports PH_ERR_TIMEOUT once, and the
 * device stays usable.  Returns PH_OK when the launch was enqueued.                  */
PH_API int phobos_selftest_bounded_wait(uint64_t limit_ns, void *stream);

/* ---- kda (chunkwise gated linear attention) ------------------------------------------- *
 * One head: Q, K, V, O [N, 64] f32, G [N, 1] the per-token log forget-gate, scale on the
 * queries (examples/kda_fp32.ph:20-65; builtins cumsum / tril / transpose, SPEC.md).  A single
 * program, as the kernel has no program_id: state S [64, 64] carried over chunks of 64 tokens. */
PH_API int phobos_kda(const PhTensor *Q, const PhTensor *K, const PhTensor *V, const PhTensor *G, const PhTensor *O,
                      float scale, void *stream);

/* ---- saxpy ------------------------------------------------------------------------- *
 * out = alpha * x + y on rank-1 f32 tensors (examples/saxpy_fp32.ph:1-5; launch shape of
 * phobos-bench/src/main.rs:1222-1236).  A rounded multiply, then a rounded add, as the
 * reference's own check computes it (main.rs:1179-1188).                                 */
PH_API int phobos_saxpy(const PhTensor *x, const PhTensor *y, const PhTensor *out, float alpha, void *stream);

/* ---- launch by entry name -------------------------------------------------- *
 * The COMPUTE operand model: Op::Compute{kernel, args, scalars, grid, cta}
 * (phobos-cluster/src/isa.rs:38-44).  `entry` is the PTX entry name the
 * reference would look up (= kernel name, phobos-lang/src/codegen/kernel.rs:90-93):
 * "gemm", "matmul", "matmul_init", "flash_attention", "saxpy", "kda".  Tensors are in
 * signature order; scalars carry their parameter position.  `grid` and `cta`
 * describe the reference's own device tiling and are validated for presence
 * only.  The GEMM regime follows from the element types unless `kind_hint`
 * (a PhGemmKind, or -1) says otherwise.  In a cluster plan "gemm" / "matmul" is
 * the accumulate STEP leaf, C = alpha*(A@B) + C, which carries the kernel's
 * scalar list but no longer uses beta (rewrite_step_store, phobos-cluster/src/
 * clustergen.rs:1363-1399): pass `(kind or PH_KIND_AUTO) | PH_LAUNCH_STEP_LEAF`
 * for it.  The executor does so by itself for a kernel whose `<name>_init` leaf is
 * registered too.                                                              */
#define PH_KIND_AUTO 0xFF
#define PH_LAUNCH_STEP_LEAF 0x100
PH_API int phobos_launch(const char *entry, const PhTensor *tensors, int32_t n_tensors, const PhScalar *scalars,
                         int32_t n_scalars, const uint32_t grid[3], const uint32_t cta[3], int32_t kind_hint,
                         void *workspace, size_t workspace_bytes, void *stream);
PH_API size_t phobos_launch_workspace_bytes(const char *entry, const PhTensor *tensors, int32_t n_tensors,
                                            int32_t kind_hint);

/* ---- input generator -------------------------------------------------------- *
 * `phobos-tensor init --fill random --seed S` (phobos-cluster/src/bin/
 * phobos-tensor.rs:55-72) = Lcg::unit_f32s (phobos-base/src/rng.rs:9-25):
 * out[i] = scale * (f32(state_i >> 33) / 2^31 - 1), element i of the stream
 * seeded with `seed`, starting at stream position `first`.  Host version
 * writes host memory; device version fills device memory (f32, or f16 with
 * the f32 value rounded RN-even) on `stream`.  `normal` != 0 draws N(0,1) by
 * Box-Muller over stream pairs instead (no reference counterpart).            */
PH_API int phobos_fill_random_host(float *out, uint64_t n, uint64_t seed, uint64_t first, float scale);
PH_API int phobos_fill_random_device(void *out, int32_t dtype, uint64_t n, uint64_t seed, uint64_t first,
                                     float scale, int32_t normal, void *stream);
/* A rows x cols block of a larger row-major tensor whose element (i, j) is
 * stream element i*stream_pitch + j: out[r*ld_out + c] takes stream element
 * first + r*stream_pitch + c (a region of the tensor `phobos-tensor init` writes). */
PH_API int phobos_fill_random_block(void *out, int32_t dtype, uint64_t rows, uint64_t cols, uint64_t ld_out,
                                    uint64_t seed, uint64_t first, uint64_t stream_pitch, float scale, void *stream);
/* f32 -> f16 (RN-even) and back on the device; element counts. */
PH_API int phobos_convert_f32_to_f16(const float *in, void *out_f16, uint64_t n, void *stream);
PH_API int phobos_convert_f16_to_f32(const void *in_f16, float *out, uint64_t n, void *stream);

/* ---- tile ids ---------------------------------------------------------------- *
 * id = (tensor:12 << 52) | (version:16 << 36) | coord:36, phobos-cluster/src/tile.rs:5-30 */
PH_API uint64_t phobos_tile_id(uint32_t tensor, uint32_t version, uint64_t coord);
PH_API uint32_t phobos_tile_tensor(uint64_t id);
PH_API uint32_t phobos_tile_version(uint64_t id);
PH_API uint64_t phobos_tile_coord(uint64_t id);
/* arena size class: phobos-pod/src/tile_store.rs:25-27 */
PH_API uint64_t phobos_size_class(uint64_t bytes);

/* ---- job file ------------------------------------------------------------------ *
 * Grammar of phobos-sched/src/job.rs:5-88: `source = <path>`, `dim NAME = INT`,
 * `tensor NAME = read|write|rmw DTYPE D0xD1 URI`, `scalar NAME = DTYPE VALUE`,
 * `#` comments.  The source file is opened only to read the kernel's name.    */
typedef struct PhJob PhJob;
typedef enum PhAccessMode { PH_READ = 0, PH_WRITE = 1, PH_RMW = 2 } PhAccessMode; /* tile.rs:86-91 */
PH_API PhJob *phobos_job_parse(const char *path);               /* NULL on error */
PH_API PhJob *phobos_job_parse_text(const char *text, const char *origin, const char *source_text);
PH_API void phobos_job_free(PhJob *job);
PH_API const char *phobos_job_kernel_name(const PhJob *job);
PH_API const char *phobos_job_source(const PhJob *job);   /* text of the `source =` file */
PH_API int32_t phobos_job_n_dims(const PhJob *job);
PH_API const char *phobos_job_dim_name(const PhJob *job, int32_t i);
PH_API int64_t phobos_job_dim_value(const PhJob *job, int32_t i);
PH_API int32_t phobos_job_n_tensors(const PhJob *job);
PH_API const char *phobos_job_tensor_name(const PhJob *job, int32_t i);
PH_API int32_t phobos_job_tensor_dtype(const PhJob *job, int32_t i);
PH_API int32_t phobos_job_tensor_mode(const PhJob *job, int32_t i);
PH_API int32_t phobos_job_tensor_rank(const PhJob *job, int32_t i);
PH_API int64_t phobos_job_tensor_dim(const PhJob *job, int32_t i, int32_t d);
PH_API const char *phobos_job_tensor_uri(const PhJob *job, int32_t i);
PH_API int32_t phobos_job_n_scalars(const PhJob *job);
PH_API const char *phobos_job_scalar_name(const PhJob *job, int32_t i);
PH_API int32_t phobos_job_scalar_dtype(const PhJob *job, int32_t i);
PH_API uint64_t phobos_job_scalar_bits(const PhJob *job, int32_t i);

/* ---- storage -------------------------------------------------------------------- *
 * file:// tensors: headerless little-endian row-major blobs; a region LOAD
 * gathers row spans into a contiguous tile and a region STORE scatters them
 * back without truncating the file (phobos-cluster/src/storage.rs:9-79).  The
 * reference is f32-only; `elem_bytes` generalises it.                          */
typedef struct PhRegion {
  int32_t rank;
  uint64_t offset[2];
  uint64_t shape[2];
} PhRegion;
PH_API int phobos_storage_path(const char *uri, char *out, size_t out_len);
PH_API int phobos_storage_load(const char *uri, const uint64_t *tensor_shape, int32_t tensor_rank,
                               const PhRegion *region, size_t elem_bytes, void *host_out);
PH_API int phobos_storage_store(const char *uri, const uint64_t *tensor_shape, int32_t tensor_rank,
                                const PhRegion *region, size_t elem_bytes, const void *host_in);

/* ---- instruction executor ----------------------------------------------------------- *
 * One executor per device: the pod's Engine (phobos-pod/src/engine.rs:121-232)
 * without the network.  Instructions carry ids and dependency lists
 * (isa.rs:52-63); an instruction is issued when all its deps have completed
 * (engine.rs:282-323, 777-789).  Ops: isa.rs:24-50.                            */
typedef enum PhOpCode { PH_OP_ALLOC = 0, PH_OP_LOAD = 1, PH_OP_FETCH = 2, PH_OP_COMPUTE = 3, PH_OP_STORE = 4,
                        PH_OP_FREE = 5 } PhOpCode;

typedef struct PhTileArg { uint64_t tile; int32_t mode; /* PhAccessMode */ } PhTileArg;

typedef struct PhInstr {
  uint64_t iid;
  const uint64_t *deps;
  int32_t n_deps;
  int32_t op;                 /* PhOpCode */
  uint64_t tile;              /* ALLOC, LOAD, FETCH, STORE, FREE */
  int32_t data_type;          /* ALLOC */
  int32_t shape_rank;         /* ALLOC */
  uint64_t shape[2];          /* ALLOC */
  uint32_t tensor;            /* LOAD/STORE: index into the tensor table (StorageRef::Tensor, isa.rs:19-22) */
  PhRegion region;            /* LOAD/STORE */
  uint32_t from_node;         /* FETCH: peer executor id */
  uint32_t kernel;            /* COMPUTE: index into the kernel table */
  const PhTileArg *args;      /* COMPUTE */
  int32_t n_args;
  const PhScalar *scalars;    /* COMPUTE */
  int32_t n_scalars;
  uint32_t grid[3], cta[3];   /* COMPUTE (validated, not used for tiling) */
  uint32_t expected_serves;   /* FREE */
} PhInstr;

typedef struct PhTensorMeta { /* phobos-pod/src/engine.rs:22-27 */
  const char *uri;
  int32_t dtype;
  int32_t rank;
  uint64_t shape[2];
  int32_t mode;
} PhTensorMeta;

typedef struct PhCompletion { uint64_t iid; uint32_t status; uint64_t elapsed_ns; } PhCompletion; /* engine.rs:70 */

typedef struct PhExecutor PhExecutor;
PH_API PhExecutor *phobos_executor_create(int32_t device, uint32_t node_id, uint64_t arena_bytes); /* NULL on error */
PH_API void phobos_executor_destroy(PhExecutor *ex);
PH_API int phobos_executor_set_tensors(PhExecutor *ex, const PhTensorMeta *tensors, int32_t n);   /* EngineMsg::SetTensors */
PH_API int phobos_executor_set_kernel(PhExecutor *ex, uint32_t kernel_id, const char *entry, int32_t kind_hint); /* SetKernels */
PH_API int phobos_executor_connect_peer(PhExecutor *ex, uint32_t node_id, PhExecutor *peer);      /* NodeAddrs/FetchLocs */
PH_API int phobos_executor_issue(PhExecutor *ex, const PhInstr *instrs, int32_t n);               /* EngineMsg::Issue(Segment) */
/* Runs the issue/poll loop until no instruction is pending or in flight.
 * Returns 0, or the status of the first failed instruction (engine.rs:744-750). */
PH_API int phobos_executor_run(PhExecutor *ex);
PH_API int32_t phobos_executor_drain_completions(PhExecutor *ex, PhCompletion *out, int32_t cap);
/* Device time of the last successful phobos_executor_run in milliseconds: from an event recorded on the
 * executor's device when the run started to the last operation it enqueued on any of its streams (CUDA events,
 * not the host clock; the reference reports elapsed_ns = 0, phobos-pod/src/engine.rs:790).  -1 before any run. */
PH_API float phobos_executor_last_run_ms(const PhExecutor *ex);
PH_API uint64_t phobos_executor_arena_used(const PhExecutor *ex);
PH_API uint64_t phobos_executor_served_bytes(const PhExecutor *ex);  /* phobos-pod/src/server.rs:22 */
/* Device address and residency of a tile (TileStore::addr/is_resident, tile_store.rs:134-140). */
PH_API int phobos_executor_tile_addr(const PhExecutor *ex, uint64_t tile, void **addr_out, int32_t *resident_out);

/* ---- `.ph` declarations and the cluster view of a kernel ------------------------------ *
 * phobos_program_parse reads the attributes, name and parameter list of kernel
 * `kernel_index` of a source text (grammar SPEC.md:5-58; phobos-lang/src/ast.rs:44-92)
 * and, when the kernel carries `@cluster`, derives what phobos-cluster/src/
 * clustergen.rs derives from it: supertile symbols per tensor axis, grid axes, access
 * modes, the accumulate-step and init leaves (or the single leaf), scalar positions.
 * No code is generated; the body is only scanned for slices and the final store.      */
typedef struct PhProgram PhProgram;
PH_API PhProgram *phobos_program_parse(const char *source_text, int32_t kernel_index);  /* NULL on error */
PH_API void phobos_program_free(PhProgram *p);
PH_API const char *phobos_program_kernel_name(const PhProgram *p);
PH_API int32_t phobos_program_n_params(const PhProgram *p);
PH_API const char *phobos_program_param_name(const PhProgram *p, int32_t i);
PH_API int32_t phobos_program_param_is_tensor(const PhProgram *p, int32_t i);
PH_API int32_t phobos_program_param_dtype(const PhProgram *p, int32_t i);
PH_API int32_t phobos_program_param_rank(const PhProgram *p, int32_t i);
PH_API const char *phobos_program_param_dim(const PhProgram *p, int32_t i, int32_t axis, int64_t *literal);
PH_API int32_t phobos_program_n_attrs(const PhProgram *p);
PH_API const char *phobos_program_attr_name(const PhProgram *p, int32_t i);
PH_API int32_t phobos_program_has_attr(const PhProgram *p, const char *attr);
/* expanded choices of `NAME in [..]` (two values = doubling steps, ast.rs:58-72) */
PH_API int32_t phobos_program_search_choices(const PhProgram *p, const char *attr, const char *dim, int64_t *out,
                                             int32_t cap);
PH_API int32_t phobos_program_is_clustered(const PhProgram *p);   /* 0: see phobos_last_error */
PH_API const char *phobos_program_describe(const PhProgram *p);   /* canonical text of the cluster program */
PH_API int32_t phobos_program_n_leaves(const PhProgram *p);
PH_API const char *phobos_program_leaf_entry(const PhProgram *p, int32_t i);   /* "<name>", "<name>_init" */
PH_API int32_t phobos_program_n_tensors(const PhProgram *p);
PH_API int32_t phobos_program_tensor_mode(const PhProgram *p, int32_t i);
/* job-file bindings against the kernel signature (names, element types, ranks, dims, scalars) */
PH_API int phobos_job_check(const PhJob *job, const PhProgram *p);

/* ---- supertile planner ------------------------------------------------------------------ *
 * plan / plan_with / plan_budgeted_with and recover_plan of phobos-sched/src/lib.rs:
 * 99-234: owner-computes placement of every output supertile (linear index modulo the
 * live nodes), tiles allocated at first use and stored / freed at last use, inputs from
 * storage (policy 0, DirectLoad) or from the lowest-numbered consumer (policy 1,
 * HomeLoadPeerFetch), segments cut by a memory budget.  The instructions are PhInstr
 * records the executor takes as they are.                                              */
typedef struct PhPlanRequest PhPlanRequest;
typedef struct PhPlan PhPlan;
PH_API PhPlanRequest *phobos_plan_request_new(uint32_t nodes, uint64_t budget_bytes, int32_t policy);
PH_API void phobos_plan_request_free(PhPlanRequest *r);
PH_API void phobos_plan_request_dim(PhPlanRequest *r, const char *name, int64_t value);
PH_API void phobos_plan_request_super(PhPlanRequest *r, const char *name, int64_t value);
PH_API void phobos_plan_request_scalar(PhPlanRequest *r, const char *name, int32_t dtype, uint64_t bits);
PH_API void phobos_plan_request_default_supers(PhPlanRequest *r, const PhProgram *p);   /* first @cluster choice */
/* turns the request into a recovery: `nodes` is the cluster width, `dead` every failed node,
 * durable (tensor, linear index) pairs are not recomputed (lib.rs:172-234) */
PH_API void phobos_plan_request_recover(PhPlanRequest *r, const uint32_t *dead, int32_t n_dead,
                                        const uint32_t *durable_tensor, const uint64_t *durable_lin, int32_t n_durable,
                                        uint16_t version, uint64_t iid_base);
PH_API PhPlan *phobos_plan_make(const PhProgram *p, const PhPlanRequest *r);   /* NULL on error */
PH_API void phobos_plan_free(PhPlan *pl);
PH_API int phobos_plan_validate(const PhPlan *pl);                             /* lib.rs:950-974 */
PH_API uint32_t phobos_plan_n_nodes(const PhPlan *pl);
PH_API int32_t phobos_plan_n_segments(const PhPlan *pl, uint32_t node);
PH_API uint64_t phobos_plan_segment_id(const PhPlan *pl, uint32_t node, int32_t seg);
PH_API int32_t phobos_plan_segment_n_instrs(const PhPlan *pl, uint32_t node, int32_t seg);
PH_API const PhInstr *phobos_plan_segment_instrs(const PhPlan *pl, uint32_t node, int32_t seg);
PH_API void phobos_plan_segment_mem(const PhPlan *pl, uint32_t node, int32_t seg, uint64_t *peak, uint64_t *incremental);
PH_API uint64_t phobos_plan_fetch_bytes(const PhPlan *pl);
PH_API uint64_t phobos_plan_peak_resident(const PhPlan *pl);
PH_API uint64_t phobos_plan_max_iid(const PhPlan *pl);
PH_API int32_t phobos_plan_n_stores(const PhPlan *pl);
PH_API void phobos_plan_store(const PhPlan *pl, int32_t i, uint64_t *iid, uint32_t *node, uint32_t *tensor, uint64_t *lin);
PH_API int32_t phobos_plan_super_shape(const PhPlan *pl, uint32_t tensor, uint64_t *shape, uint64_t *grid, int32_t cap);
PH_API int32_t phobos_plan_owner(const PhPlan *pl, uint32_t tensor, uint64_t lin);   /* -1: not in this plan */

/* Ranks every combination of the @cluster choices by the makespan of its plan: busiest
 * node's flops / leaf rate against busiest node's fetched bytes / link rate; configs that
 * leave a node idle or exceed `vram_bytes` are dropped (phobos-sched/src/autotune.rs:40-192). */
typedef struct PhTuneResult PhTuneResult;
PH_API PhTuneResult *phobos_autotune(const PhProgram *p, const PhPlanRequest *dims_from, uint32_t nodes,
                                     uint64_t vram_bytes, double link_bytes_per_sec, double leaf_flops_per_sec);
PH_API void phobos_autotune_free(PhTuneResult *r);
PH_API int32_t phobos_autotune_n(const PhTuneResult *r);
PH_API int64_t phobos_autotune_super(const PhTuneResult *r, int32_t i, const char *name);
PH_API void phobos_autotune_cost(const PhTuneResult *r, int32_t i, double *makespan, double *compute, double *comm,
                                 uint64_t *peak, uint64_t *fetch_bytes);

/* ---- wire format of segments --------------------------------------------------------------- *
 * `phobos.v1.Segment` (phobos-cluster/proto/v1/phobos_v1_isa.proto:93-113) to and from PhInstr
 * records, without a protobuf runtime: segments a phobos scheduler emits can be issued to the
 * executor, and segments planned here can be sent to a phobos pod.                            */
typedef struct PhSegmentMsg PhSegmentMsg;
PH_API PhSegmentMsg *phobos_segment_decode(const void *data, size_t n);   /* NULL on error */
PH_API void phobos_segment_free(PhSegmentMsg *m);
PH_API uint64_t phobos_segment_id(const PhSegmentMsg *m);
PH_API int32_t phobos_segment_n_instrs(const PhSegmentMsg *m);
PH_API const PhInstr *phobos_segment_instrs(const PhSegmentMsg *m);
/* encoded size (written to `out` when `cap` suffices); SIZE_MAX on error */
PH_API size_t phobos_segment_encode(uint64_t id, const PhInstr *instrs, int32_t n, void *out, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* PHOBOS_LEAF_H_ */
