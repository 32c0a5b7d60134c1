"""Python host side of the B200 leaf executor for phobos kernels.

A thin ctypes mirror of ``include/phobos_leaf.h``: the same entry points, the
same argument meaning and error behaviour as the reference's leaf launch
interface (``launch_gemm`` / ``launch_flash`` in phobos-bench/src/main.rs:290-371
and the pod's COMPUTE in phobos-pod/src/engine.rs:542-653).  torch is used for
device memory and streams only; every computation runs in ``libphobos_leaf.so``
(hand-written sm_100a CUDA).  There is no CPU or eager fallback: if the shared
library is missing, loading this package's native side raises.
"""
from __future__ import annotations

import ctypes
import struct
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libphobos_leaf.so"

# ---- enums (include/phobos_leaf.h) ----------------------------------------------------
PH_OK, PH_ERR_INVALID, PH_ERR_UNSUPPORTED, PH_ERR_DEVICE = 0, -1, -2, -3
PH_ERR_WORKSPACE, PH_ERR_TIMEOUT, PH_ERR_IO, PH_ERR_PARSE, PH_ERR_STATE = -4, -5, -6, -7, -8
F16, F32, F64, I8, I32, I64, BOOL = range(7)
GEMM_FP32, GEMM_FP16TC_FP32ACC, GEMM_FP16 = 0, 1, 2
READ, WRITE, RMW = 0, 1, 2
OP_ALLOC, OP_LOAD, OP_FETCH, OP_COMPUTE, OP_STORE, OP_FREE = range(6)
DTYPE_NAMES = {F16: "f16", F32: "f32", F64: "f64", I8: "i8", I32: "i32", I64: "i64", BOOL: "bool"}


class PhobosError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


class PhTensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("sizes", ctypes.c_int64 * 2), ("strides", ctypes.c_int64 * 2), ("offset", ctypes.c_int64)]


class PhScalar(ctypes.Structure):
    _fields_ = [("pos", ctypes.c_uint32), ("dtype", ctypes.c_int32), ("bits", ctypes.c_uint64)]


class PhDeviceInfo(ctypes.Structure):
    _fields_ = [("device", ctypes.c_int32), ("sm_count", ctypes.c_int32), ("cc_major", ctypes.c_int32),
                ("cc_minor", ctypes.c_int32), ("sm_clock_khz", ctypes.c_int32), ("total_mem_bytes", ctypes.c_int64),
                ("fp32_peak_flops", ctypes.c_double), ("name", ctypes.c_char * 64)]


class PhRegion(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int32), ("offset", ctypes.c_uint64 * 2), ("shape", ctypes.c_uint64 * 2)]


class PhTileArg(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_uint64), ("mode", ctypes.c_int32)]


class PhInstr(ctypes.Structure):
    _fields_ = [("iid", ctypes.c_uint64), ("deps", ctypes.POINTER(ctypes.c_uint64)), ("n_deps", ctypes.c_int32),
                ("op", ctypes.c_int32), ("tile", ctypes.c_uint64), ("data_type", ctypes.c_int32),
                ("shape_rank", ctypes.c_int32), ("shape", ctypes.c_uint64 * 2), ("tensor", ctypes.c_uint32),
                ("region", PhRegion), ("from_node", ctypes.c_uint32), ("kernel", ctypes.c_uint32),
                ("args", ctypes.POINTER(PhTileArg)), ("n_args", ctypes.c_int32),
                ("scalars", ctypes.POINTER(PhScalar)), ("n_scalars", ctypes.c_int32),
                ("grid", ctypes.c_uint32 * 3), ("cta", ctypes.c_uint32 * 3), ("expected_serves", ctypes.c_uint32)]


class PhTensorMeta(ctypes.Structure):
    _fields_ = [("uri", ctypes.c_char_p), ("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_uint64 * 2), ("mode", ctypes.c_int32)]


class PhCompletion(ctypes.Structure):
    _fields_ = [("iid", ctypes.c_uint64), ("status", ctypes.c_uint32), ("elapsed_ns", ctypes.c_uint64)]


_lib = None


def lib() -> ctypes.CDLL:
    """The native library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python phobos-lang_b200/build.py` "
                              "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the leaf kernels.")
        L = ctypes.CDLL(str(LIB_PATH))
        c = ctypes
        vp, i32, i64, u32, u64, f32, sz = c.c_void_p, c.c_int32, c.c_int64, c.c_uint32, c.c_uint64, c.c_float, c.c_size_t
        TP, SP = c.POINTER(PhTensor), c.POINTER(PhScalar)
        sigs = {
            "phobos_last_error": (c.c_char_p, []),
            "phobos_version": (c.c_char_p, []),
            "phobos_dtype_bytes": (sz, [i32]),
            "phobos_device_info": (c.c_int, [c.c_int, c.POINTER(PhDeviceInfo)]),
            "phobos_device_status": (c.c_int, [vp, c.POINTER(u32)]),
            "phobos_gemm": (c.c_int, [TP, TP, TP, f32, f32, i32, vp, sz, vp]),
            "phobos_saxpy": (c.c_int, [TP, TP, TP, f32, vp]),
            "phobos_kda": (c.c_int, [TP, TP, TP, TP, TP, f32, vp]),
            "phobos_gemm_workspace_bytes": (sz, [i32, i32, i64, i64, i64]),
            "phobos_gemm_fp16tc_noalloc": (c.c_int, [TP, TP, TP, f32, f32, vp]),
            "phobos_matmul_init": (c.c_int, [TP, f32, i32, vp]),
            "phobos_flash_attention": (c.c_int, [TP, TP, TP, TP, f32, i64, vp, sz, vp]),
            "phobos_flash_workspace_bytes": (sz, [i32, i64, i64, i64, i64]),
            "phobos_last_launch_clock": (c.c_int, [vp, c.POINTER(u64), c.POINTER(u64)]),
            "phobos_selftest_bounded_wait": (c.c_int, [u64, vp]),
            "phobos_launch": (c.c_int, [c.c_char_p, TP, i32, SP, i32, c.POINTER(u32), c.POINTER(u32), i32, vp, sz, vp]),
            "phobos_launch_workspace_bytes": (sz, [c.c_char_p, TP, i32, i32]),
            "phobos_fill_random_host": (c.c_int, [c.POINTER(f32), u64, u64, u64, f32]),
            "phobos_fill_random_device": (c.c_int, [vp, i32, u64, u64, u64, f32, i32, vp]),
            "phobos_fill_random_block": (c.c_int, [vp, i32, u64, u64, u64, u64, u64, u64, f32, vp]),
            "phobos_convert_f32_to_f16": (c.c_int, [vp, vp, u64, vp]),
            "phobos_convert_f16_to_f32": (c.c_int, [vp, vp, u64, vp]),
            "phobos_tile_id": (u64, [u32, u32, u64]),
            "phobos_tile_tensor": (u32, [u64]),
            "phobos_tile_version": (u32, [u64]),
            "phobos_tile_coord": (u64, [u64]),
            "phobos_size_class": (u64, [u64]),
            "phobos_job_parse": (vp, [c.c_char_p]),
            "phobos_job_parse_text": (vp, [c.c_char_p, c.c_char_p, c.c_char_p]),
            "phobos_job_free": (None, [vp]),
            "phobos_job_kernel_name": (c.c_char_p, [vp]),
            "phobos_job_source": (c.c_char_p, [vp]),
            "phobos_job_n_dims": (i32, [vp]),
            "phobos_job_dim_name": (c.c_char_p, [vp, i32]),
            "phobos_job_dim_value": (i64, [vp, i32]),
            "phobos_job_n_tensors": (i32, [vp]),
            "phobos_job_tensor_name": (c.c_char_p, [vp, i32]),
            "phobos_job_tensor_dtype": (i32, [vp, i32]),
            "phobos_job_tensor_mode": (i32, [vp, i32]),
            "phobos_job_tensor_rank": (i32, [vp, i32]),
            "phobos_job_tensor_dim": (i64, [vp, i32, i32]),
            "phobos_job_tensor_uri": (c.c_char_p, [vp, i32]),
            "phobos_job_n_scalars": (i32, [vp]),
            "phobos_job_scalar_name": (c.c_char_p, [vp, i32]),
            "phobos_job_scalar_dtype": (i32, [vp, i32]),
            "phobos_job_scalar_bits": (u64, [vp, i32]),
            "phobos_storage_path": (c.c_int, [c.c_char_p, c.c_char_p, sz]),
            "phobos_storage_load": (c.c_int, [c.c_char_p, c.POINTER(u64), i32, c.POINTER(PhRegion), sz, vp]),
            "phobos_storage_store": (c.c_int, [c.c_char_p, c.POINTER(u64), i32, c.POINTER(PhRegion), sz, vp]),
            "phobos_executor_create": (vp, [i32, u32, u64]),
            "phobos_executor_destroy": (None, [vp]),
            "phobos_executor_set_tensors": (c.c_int, [vp, c.POINTER(PhTensorMeta), i32]),
            "phobos_executor_set_kernel": (c.c_int, [vp, u32, c.c_char_p, i32]),
            "phobos_executor_connect_peer": (c.c_int, [vp, u32, vp]),
            "phobos_executor_issue": (c.c_int, [vp, c.POINTER(PhInstr), i32]),
            "phobos_executor_run": (c.c_int, [vp]),
            "phobos_executor_drain_completions": (i32, [vp, c.POINTER(PhCompletion), i32]),
            "phobos_executor_last_run_ms": (c.c_float, [vp]),
            "phobos_executor_arena_used": (u64, [vp]),
            "phobos_executor_served_bytes": (u64, [vp]),
            "phobos_executor_tile_addr": (c.c_int, [vp, u64, c.POINTER(vp), c.POINTER(i32)]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(L, name)  # AttributeError here means the library is stale: rebuild
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().phobos_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise PhobosError(rc, last_error())


# ---- descriptors ----------------------------------------------------------------------
def _torch_dtype_code(t) -> int:
    import torch
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.float32:
        return F32
    raise PhobosError(PH_ERR_UNSUPPORTED, f"element type {t.dtype} is not f16 or f32")


def tensor_desc(t) -> PhTensor:
    """PhTensor for a rank-1/2 CUDA torch tensor (no copy; the caller keeps `t` alive)."""
    if not t.is_cuda:
        raise PhobosError(PH_ERR_INVALID, "tensor is not on a CUDA device")
    import torch
    if t.device.index != torch.cuda.current_device():
        # the library launches on the current device and uses that device's status word
        raise PhobosError(PH_ERR_INVALID, f"tensor lives on cuda:{t.device.index} but the current device is "
                                          f"cuda:{torch.cuda.current_device()}")
    d = PhTensor()
    d.ptr = t.data_ptr()
    d.dtype = _torch_dtype_code(t)
    d.rank = t.dim()
    if t.dim() not in (1, 2):
        raise PhobosError(PH_ERR_INVALID, f"rank {t.dim()}, expected 1 or 2")
    for i in range(t.dim()):
        d.sizes[i] = t.shape[i]
        d.strides[i] = t.stride(i)
    d.offset = 0
    return d


def raw_desc(ptr: int, dtype: int, rows: int, cols: int, ld: int | None = None, offset: int = 0) -> PhTensor:
    d = PhTensor()
    d.ptr = ptr
    d.dtype = dtype
    d.rank = 2
    d.sizes[0], d.sizes[1] = rows, cols
    d.strides[0], d.strides[1] = (cols if ld is None else ld), 1
    d.offset = offset
    return d


def scalar_f32(pos: int, value: float) -> PhScalar:
    """ScalarArg{pos, F32(value)} with the to_bits encoding (phobos-cluster/src/tile.rs:75-83)."""
    return PhScalar(pos, F32, struct.unpack("<I", struct.pack("<f", value))[0])


def _stream_ptr(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _ws(workspace):
    if workspace is None:
        return None, 0
    return workspace.data_ptr(), workspace.numel() * workspace.element_size()


# ---- leaf kernels ---------------------------------------------------------------------------
def gemm(A, B, C, alpha: float, beta: float, kind: int, workspace=None, stream=None) -> None:
    """C = alpha * A@B + beta * C, in place on C (launch_gemm, phobos-bench/src/main.rs:290-327)."""
    a, b, c = tensor_desc(A), tensor_desc(B), tensor_desc(C)
    wp, wn = _ws(workspace)
    check(lib().phobos_gemm(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), alpha, beta, kind, wp, wn,
                            _stream_ptr(stream)))


NOALLOC_SCRATCH_BYTES = 8 << 20
KIND_AUTO = 0xFF            # kind_hint: regime from the element types ...
LAUNCH_STEP_LEAF = 0x100     # ... | this: gemm/matmul is the accumulate step of a cluster chain (beta unused)


def gemm_fp16tc_noalloc(A, B, C, alpha: float, beta: float, stream=None) -> None:
    """gemm_fp16tc_fp32acc on f32-stored A, B, C without a caller workspace and without any allocation.

    For callers that cannot lend scratch memory and may not allocate it (a pod whose device budget is
    all in its tile arena, a loop barred from the CUDA allocator): the rounded f16 copies of A and B
    go to a fixed NOALLOC_SCRATCH_BYTES array inside the library, so 2*(M*K + K*N) bytes must fit.
    All calls on a device share that array: do not let two of them overlap on the GPU.
    """
    a, b, c = tensor_desc(A), tensor_desc(B), tensor_desc(C)
    check(lib().phobos_gemm_fp16tc_noalloc(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), alpha, beta,
                                           _stream_ptr(stream)))


def kda(Q, K, V, G, O, scale: float, stream=None) -> None:
    """Chunkwise gated linear attention of one head (examples/kda_fp32.ph): Q, K, V, O [N, 64], G [N, 1]."""
    d = [tensor_desc(t) for t in (Q, K, V, G, O)]
    check(lib().phobos_kda(*(ctypes.byref(x) for x in d), scale, _stream_ptr(stream)))


def saxpy(x, y, out, alpha: float, stream=None) -> None:
    """out = alpha * x + y on rank-1 f32 tensors (examples/saxpy_fp32.ph; phobos-bench/src/main.rs:1190-1250)."""
    dx, dy, do = tensor_desc(x), tensor_desc(y), tensor_desc(out)
    check(lib().phobos_saxpy(ctypes.byref(dx), ctypes.byref(dy), ctypes.byref(do), alpha, _stream_ptr(stream)))


def gemm_workspace_bytes(kind: int, a_dtype: int, M: int, N: int, K: int) -> int:
    return int(lib().phobos_gemm_workspace_bytes(kind, a_dtype, M, N, K))


def matmul_init(C, beta: float, zero_fill: bool = False, stream=None) -> None:
    """The `<kernel>_init` leaf: C = beta*C or C = 0 (phobos-cluster/src/clustergen.rs:1276-1360)."""
    c = tensor_desc(C)
    check(lib().phobos_matmul_init(ctypes.byref(c), beta, int(zero_fill), _stream_ptr(stream)))


def flash_attention(Q, K, V, O, scale: float, workspace=None, stream=None) -> None:
    """O = softmax(scale * Q K^T) V per (batch*head) slab (launch_flash, main.rs:334-371).

    Q, O: [Nq, D] or [BH, Nq, D]; K, V: [Nk, D] or [BH, Nk, D]; contiguous.
    """
    bh = 1
    if Q.dim() == 3:
        bh = Q.shape[0]
        if K.shape[0] != bh or V.shape[0] != bh or O.shape[0] != bh:
            raise PhobosError(PH_ERR_INVALID, "batch*head extents differ")
        for t in (Q, K, V, O):
            if not t.is_contiguous():
                raise PhobosError(PH_ERR_INVALID, "flash_attention: tensors must be contiguous [BH, N, D]")
        q, k, v, o = (tensor_desc(t[0]) for t in (Q, K, V, O))
    else:
        q, k, v, o = (tensor_desc(t) for t in (Q, K, V, O))
    wp, wn = _ws(workspace)
    check(lib().phobos_flash_attention(ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(o), scale, bh,
                                       wp, wn, _stream_ptr(stream)))


def flash_workspace_bytes(dtype: int, batch_heads: int, Nq: int, Nk: int, D: int) -> int:
    return int(lib().phobos_flash_workspace_bytes(dtype, batch_heads, Nq, Nk, D))


def launch(entry: str, tensors, scalars, grid=(1, 1, 1), cta=(256, 1, 1), kind_hint: int = -1, workspace=None,
           stream=None) -> None:
    """COMPUTE by entry name (Op::Compute, phobos-cluster/src/isa.rs:38-44)."""
    descs = (PhTensor * len(tensors))(*[tensor_desc(t) for t in tensors])
    sc = (PhScalar * max(1, len(scalars)))(*scalars)
    g = (ctypes.c_uint32 * 3)(*grid)
    b = (ctypes.c_uint32 * 3)(*cta)
    wp, wn = _ws(workspace)
    check(lib().phobos_launch(entry.encode(), descs, len(tensors), sc, len(scalars), g, b, kind_hint, wp, wn,
                              _stream_ptr(stream)))


def device_status(stream=None) -> int:
    """Synchronises the stream and returns (clearing) the device's wait-status word; raises on a timeout."""
    w = ctypes.c_uint32(0)
    check(lib().phobos_device_status(_stream_ptr(stream), ctypes.byref(w)))
    return int(w.value)


def last_launch_clock(stream=None) -> tuple[int, int]:
    """(SM cycles, timer nanoseconds) one CTA of the most recent GEMM / flash launch on the current device lived;
    cycles / ns is the SM clock in GHz during that launch.  Synchronises the stream."""
    cyc, ns = ctypes.c_uint64(0), ctypes.c_uint64(0)
    check(lib().phobos_last_launch_clock(_stream_ptr(stream), ctypes.byref(cyc), ctypes.byref(ns)))
    return int(cyc.value), int(ns.value)


def selftest_bounded_wait(limit_ns: int, stream=None) -> None:
    """Enqueues a one-CTA kernel whose barrier wait must run out after `limit_ns`; device_status() then raises
    PH_ERR_TIMEOUT once and the device stays usable."""
    check(lib().phobos_selftest_bounded_wait(limit_ns, _stream_ptr(stream)))


def device_info(device: int = 0) -> PhDeviceInfo:
    info = PhDeviceInfo()
    check(lib().phobos_device_info(device, ctypes.byref(info)))
    return info


# ---- generator / conversions -------------------------------------------------------------------
def fill_random(out, seed: int, first: int = 0, scale: float = 1.0, normal: bool = False, stream=None) -> None:
    """Fill a CUDA f32/f16 tensor with the Lcg stream (`phobos-tensor init --fill random --seed`)."""
    if not out.is_contiguous():
        raise PhobosError(PH_ERR_INVALID, "fill_random needs a contiguous tensor")
    check(lib().phobos_fill_random_device(out.data_ptr(), _torch_dtype_code(out), out.numel(), seed, first, scale,
                                          int(normal), _stream_ptr(stream)))


def fill_random_block(out, seed: int, first: int, stream_pitch: int, scale: float = 1.0, stream=None) -> None:
    """Fill a 2-D CUDA tensor (inner stride 1) with a block of a larger seeded tensor: element (r, c)
    takes stream element first + r*stream_pitch + c."""
    if out.dim() != 2 or out.stride(1) != 1:
        raise PhobosError(PH_ERR_INVALID, "fill_random_block needs a rank-2 tensor with inner stride 1")
    check(lib().phobos_fill_random_block(out.data_ptr(), _torch_dtype_code(out), out.shape[0], out.shape[1],
                                         out.stride(0), seed, first, stream_pitch, scale, _stream_ptr(stream)))


def fill_random_host(n: int, seed: int, first: int = 0, scale: float = 1.0):
    import numpy as np
    out = np.empty(n, dtype=np.float32)
    check(lib().phobos_fill_random_host(out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), n, seed, first, scale))
    return out


# ---- tile ids --------------------------------------------------------------------------------------
def tile_id(tensor: int, version: int, coord: int) -> int:
    return int(lib().phobos_tile_id(tensor, version, coord))


def tile_fields(tid: int) -> tuple[int, int, int]:
    L = lib()
    return int(L.phobos_tile_tensor(tid)), int(L.phobos_tile_version(tid)), int(L.phobos_tile_coord(tid))


def tile_tensor(tid: int) -> int:
    return tile_fields(tid)[0]


def tile_version(tid: int) -> int:
    return tile_fields(tid)[1]


def tile_coord(tid: int) -> int:
    return tile_fields(tid)[2]


def size_class(nbytes: int) -> int:
    return int(lib().phobos_size_class(nbytes))


from .job import Job, parse_job, parse_job_text  # noqa: E402
from .storage import load_region, storage_path, store_region  # noqa: E402
from .executor import Executor, Instr, device_uri  # noqa: E402
from .partition import PartitionPlan, plan_partition  # noqa: E402
from .hostpipe import HostPipeline  # noqa: E402
from .planner import (DIRECT_LOAD, HOME_LOAD_PEER_FETCH, NO_BUDGET, Plan, Program, autotune, decode_segment,  # noqa: E402
                      encode_segment, plan, run_plan)
