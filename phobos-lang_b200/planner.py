"""`.ph` declarations, cluster programs and supertile plans (ctypes mirror of the planner ABI).

Program  = what phobos-cluster's clustergen derives from a `@cluster` kernel
           (phobos-cluster/src/ir.rs:5-103): tensors with supertile symbols and access modes,
           scalars, leaves (step + init, or one leaf), grid axes.
plan()   = phobos_sched::plan / plan_with / plan_budgeted_with / recover_plan
           (phobos-sched/src/lib.rs:99-234): per-node segments of executor instructions.
autotune = phobos_sched::autotune::autotune (phobos-sched/src/autotune.rs:40-97).
run_plan = what the scheduler's dispatch loop does with a plan on one box: one executor per
           node, every segment issued in order, all executors driven to completion.
"""
from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass

DIRECT_LOAD = 0            # IngestPolicy::DirectLoad (default)
HOME_LOAD_PEER_FETCH = 1   # IngestPolicy::HomeLoadPeerFetch
NO_BUDGET = (1 << 64) - 1


def _L():
    from . import lib
    L = lib()
    if getattr(L, "_plan_sigs", False):
        return L
    c = ctypes
    vp, i32, i64, u32, u64, cp = c.c_void_p, c.c_int32, c.c_int64, c.c_uint32, c.c_uint64, c.c_char_p
    sig = {
        "phobos_program_parse": (vp, [cp, i32]), "phobos_program_free": (None, [vp]),
        "phobos_program_kernel_name": (cp, [vp]), "phobos_program_n_params": (i32, [vp]),
        "phobos_program_param_name": (cp, [vp, i32]), "phobos_program_param_is_tensor": (i32, [vp, i32]),
        "phobos_program_param_dtype": (i32, [vp, i32]), "phobos_program_param_rank": (i32, [vp, i32]),
        "phobos_program_param_dim": (cp, [vp, i32, i32, c.POINTER(i64)]),
        "phobos_program_n_attrs": (i32, [vp]), "phobos_program_attr_name": (cp, [vp, i32]),
        "phobos_program_has_attr": (i32, [vp, cp]),
        "phobos_program_search_choices": (i32, [vp, cp, cp, c.POINTER(i64), i32]),
        "phobos_program_is_clustered": (i32, [vp]), "phobos_program_describe": (cp, [vp]),
        "phobos_program_n_leaves": (i32, [vp]), "phobos_program_leaf_entry": (cp, [vp, i32]),
        "phobos_program_n_tensors": (i32, [vp]), "phobos_program_tensor_mode": (i32, [vp, i32]),
        "phobos_job_check": (i32, [vp, vp]),
        "phobos_plan_request_new": (vp, [u32, u64, i32]), "phobos_plan_request_free": (None, [vp]),
        "phobos_plan_request_dim": (None, [vp, cp, i64]), "phobos_plan_request_super": (None, [vp, cp, i64]),
        "phobos_plan_request_scalar": (None, [vp, cp, i32, u64]),
        "phobos_plan_request_default_supers": (None, [vp, vp]),
        "phobos_plan_request_recover": (None, [vp, c.POINTER(u32), i32, c.POINTER(u32), c.POINTER(u64), i32, c.c_uint16, u64]),
        "phobos_plan_make": (vp, [vp, vp]), "phobos_plan_free": (None, [vp]), "phobos_plan_validate": (i32, [vp]),
        "phobos_plan_n_nodes": (u32, [vp]), "phobos_plan_n_segments": (i32, [vp, u32]),
        "phobos_plan_segment_id": (u64, [vp, u32, i32]), "phobos_plan_segment_n_instrs": (i32, [vp, u32, i32]),
        "phobos_plan_segment_instrs": (vp, [vp, u32, i32]),
        "phobos_plan_segment_mem": (None, [vp, u32, i32, c.POINTER(u64), c.POINTER(u64)]),
        "phobos_plan_fetch_bytes": (u64, [vp]), "phobos_plan_peak_resident": (u64, [vp]), "phobos_plan_max_iid": (u64, [vp]),
        "phobos_plan_n_stores": (i32, [vp]),
        "phobos_plan_store": (None, [vp, i32, c.POINTER(u64), c.POINTER(u32), c.POINTER(u32), c.POINTER(u64)]),
        "phobos_plan_super_shape": (i32, [vp, u32, c.POINTER(u64), c.POINTER(u64), i32]),
        "phobos_plan_owner": (i32, [vp, u32, u64]),
        "phobos_autotune": (vp, [vp, vp, u32, u64, c.c_double, c.c_double]), "phobos_autotune_free": (None, [vp]),
        "phobos_autotune_n": (i32, [vp]), "phobos_autotune_super": (i64, [vp, i32, cp]),
        "phobos_autotune_cost": (None, [vp, i32, c.POINTER(c.c_double), c.POINTER(c.c_double), c.POINTER(c.c_double),
                                        c.POINTER(u64), c.POINTER(u64)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    L._plan_sigs = True
    return L


@dataclass
class Param:
    name: str
    is_tensor: bool
    dtype: int
    dims: tuple = ()      # symbolic names (str) or literal extents (int)


class Program:
    """One kernel of a `.ph` source: its declaration and, under `@cluster`, its cluster program."""

    def __init__(self, source_text: str, kernel_index: int = 0):
        from . import PH_ERR_PARSE, PhobosError, last_error
        self._L = _L()
        self._h = self._L.phobos_program_parse(source_text.encode(), kernel_index)
        if not self._h:
            raise PhobosError(PH_ERR_PARSE, last_error())
        L, h = self._L, self._h
        self.name = L.phobos_program_kernel_name(h).decode()
        self.params = []
        for i in range(L.phobos_program_n_params(h)):
            dims = []
            for ax in range(max(0, L.phobos_program_param_rank(h, i)) if L.phobos_program_param_is_tensor(h, i) else 0):
                lit = ctypes.c_int64()
                sym = L.phobos_program_param_dim(h, i, ax, ctypes.byref(lit)).decode()
                dims.append(sym if lit.value < 0 else int(lit.value))
            self.params.append(Param(L.phobos_program_param_name(h, i).decode(), bool(L.phobos_program_param_is_tensor(h, i)),
                                     L.phobos_program_param_dtype(h, i), tuple(dims)))
        self.attrs = [L.phobos_program_attr_name(h, i).decode() for i in range(L.phobos_program_n_attrs(h))]
        self.clustered = bool(L.phobos_program_is_clustered(h))
        self.cluster_error = "" if self.clustered else last_error()
        self.leaves = [L.phobos_program_leaf_entry(h, i).decode() for i in range(L.phobos_program_n_leaves(h))]
        self.tensor_modes = [L.phobos_program_tensor_mode(h, i) for i in range(L.phobos_program_n_tensors(h))]

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.phobos_program_free(self._h)
            self._h = None

    def has_attr(self, name: str) -> bool:
        return bool(self._L.phobos_program_has_attr(self._h, name.encode()))

    def search_choices(self, attr: str, dim: str):
        buf = (ctypes.c_int64 * 64)()
        n = self._L.phobos_program_search_choices(self._h, attr.encode(), dim.encode(), buf, 64)
        return None if n < 0 else [int(buf[i]) for i in range(n)]

    def describe(self) -> str:
        return self._L.phobos_program_describe(self._h).decode()

    def check_job(self, job) -> None:
        """Raises when the job's tensor / scalar / dim bindings do not fit the kernel's signature."""
        from . import check
        check(self._L.phobos_job_check(job._handle, self._h))


class Plan:
    def __init__(self, L, handle):
        self._L, self._h = L, handle
        self.n_nodes = int(L.phobos_plan_n_nodes(handle))
        self.fetch_bytes = int(L.phobos_plan_fetch_bytes(handle))
        self.peak_resident = int(L.phobos_plan_peak_resident(handle))
        self.max_iid = int(L.phobos_plan_max_iid(handle))
        self.stores = []
        for i in range(L.phobos_plan_n_stores(handle)):
            iid, node, tensor, lin = ctypes.c_uint64(), ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
            L.phobos_plan_store(handle, i, ctypes.byref(iid), ctypes.byref(node), ctypes.byref(tensor), ctypes.byref(lin))
            self.stores.append((iid.value, node.value, tensor.value, lin.value))

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.phobos_plan_free(self._h)
            self._h = None

    def validate(self) -> None:
        from . import check
        check(self._L.phobos_plan_validate(self._h))

    def segments(self, node: int):
        """[(segment id, [Instr, ...], peak bytes, incremental bytes), ...] in dispatch order."""
        out = []
        for s in range(self._L.phobos_plan_n_segments(self._h, node)):
            n = self._L.phobos_plan_segment_n_instrs(self._h, node, s)
            ptr = self._L.phobos_plan_segment_instrs(self._h, node, s)
            instrs = _instrs_from_array(ptr, n)
            peak, inc = ctypes.c_uint64(), ctypes.c_uint64()
            self._L.phobos_plan_segment_mem(self._h, node, s, ctypes.byref(peak), ctypes.byref(inc))
            out.append((int(self._L.phobos_plan_segment_id(self._h, node, s)), instrs, peak.value, inc.value))
        return out

    def node_instrs(self, node: int):
        return [i for _, instrs, _, _ in self.segments(node) for i in instrs]

    def super_shape(self, tensor: int):
        shape, grid = (ctypes.c_uint64 * 4)(), (ctypes.c_uint64 * 4)()
        n = self._L.phobos_plan_super_shape(self._h, tensor, shape, grid, 4)
        return tuple(int(shape[i]) for i in range(n)), tuple(int(grid[i]) for i in range(n))

    def owner(self, tensor: int, lin: int) -> int:
        return int(self._L.phobos_plan_owner(self._h, tensor, lin))


def _copy_scalar(s):
    from . import PhScalar
    return PhScalar(int(s.pos), int(s.dtype), int(s.bits))


def _request(L, program, dims, supers, nodes, budget, policy, scalars):
    rq = L.phobos_plan_request_new(nodes, budget, policy)
    for k, v in dims.items():
        L.phobos_plan_request_dim(rq, k.encode(), int(v))
    if supers is None:
        L.phobos_plan_request_default_supers(rq, program._h)
    else:
        for k, v in supers.items():
            L.phobos_plan_request_super(rq, k.encode(), int(v))
    for name, sc in (scalars or {}).items():
        L.phobos_plan_request_scalar(rq, name.encode(), int(sc.dtype), int(sc.bits))
    return rq


def plan(program: Program, dims: dict, supers: dict | None = None, nodes: int = 1, budget: int = NO_BUDGET,
         policy: int = DIRECT_LOAD, scalars: dict | None = None, recover: dict | None = None) -> Plan:
    """scalars: name -> PhScalar (pos ignored).  recover: {"dead": [...], "durable": [(tensor, lin), ...],
    "version": v, "iid_base": n} turns the call into recover_plan with `nodes` = cluster width."""
    from . import PH_ERR_INVALID, PhobosError, last_error
    L = _L()
    rq = _request(L, program, dims, supers, nodes, budget, policy, scalars)
    try:
        if recover is not None:
            dead = list(recover.get("dead", ()))
            dur = list(recover.get("durable", ()))
            d = (ctypes.c_uint32 * max(1, len(dead)))(*dead)
            dt = (ctypes.c_uint32 * max(1, len(dur)))(*[t for t, _ in dur])
            dl = (ctypes.c_uint64 * max(1, len(dur)))(*[l for _, l in dur])
            L.phobos_plan_request_recover(rq, d, len(dead), dt, dl, len(dur), int(recover.get("version", 1)),
                                          int(recover.get("iid_base", 0)))
        h = L.phobos_plan_make(program._h, rq)
        if not h:
            raise PhobosError(PH_ERR_INVALID, last_error())
        return Plan(L, h)
    finally:
        L.phobos_plan_request_free(rq)


def autotune(program: Program, dims: dict, nodes: int, vram_bytes: int, link_bytes_per_sec: float,
             leaf_flops_per_sec: float):
    """Ranked supertile configurations, best first: dicts with supers, makespan_sec, compute_sec, comm_sec,
    peak_resident, fetch_bytes."""
    from . import PH_ERR_INVALID, PhobosError, last_error
    L = _L()
    rq = _request(L, program, dims, {}, nodes, NO_BUDGET, DIRECT_LOAD, None)
    try:
        r = L.phobos_autotune(program._h, rq, nodes, vram_bytes, link_bytes_per_sec, leaf_flops_per_sec)
        if not r:
            raise PhobosError(PH_ERR_INVALID, last_error())
    finally:
        L.phobos_plan_request_free(rq)
    try:
        names = sorted({p_ for p_ in _cluster_dims(program)})
        out = []
        for i in range(L.phobos_autotune_n(r)):
            mk, cs, cm = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
            pk, fb = ctypes.c_uint64(), ctypes.c_uint64()
            L.phobos_autotune_cost(r, i, ctypes.byref(mk), ctypes.byref(cs), ctypes.byref(cm), ctypes.byref(pk), ctypes.byref(fb))
            out.append({"supers": {n: int(L.phobos_autotune_super(r, i, n.encode())) for n in names},
                        "makespan_sec": mk.value, "compute_sec": cs.value, "comm_sec": cm.value,
                        "peak_resident": pk.value, "fetch_bytes": fb.value})
        return out
    finally:
        L.phobos_autotune_free(r)


def _cluster_dims(program: Program):
    for line in program.describe().splitlines():
        if line.startswith("super "):
            yield line.split()[1]


def run_plan(pl: Plan, program: Program, tensors, executors) -> None:
    """Runs a plan on one box: executors[n] plays node n.  tensors: [(uri, dtype, shape, mode), ...] in the
    kernel's tensor order.  Kernel ids are leaf indices; every executor knows every other as a FETCH peer."""
    for n, ex in enumerate(executors):
        ex.set_tensors(tensors)
        for k, entry in enumerate(program.leaves):
            ex.set_kernel(k, entry)
        for m, peer in enumerate(executors):
            if m != n:
                ex.connect_peer(m, peer)
    for n, ex in enumerate(executors):
        for _, instrs, _, _ in pl.segments(n):
            if instrs:
                ex.issue(instrs)
    errors = [None] * len(executors)

    def drive(n):
        try:
            executors[n].run()
        except Exception as e:  # noqa: BLE001 - reported to the caller below
            errors[n] = e

    threads = [threading.Thread(target=drive, args=(n,)) for n in range(len(executors))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for e in errors:
        if e is not None:
            raise e


# ---- wire format of segments (phobos.v1.Segment) -----------------------------------------------------
def _wire_sigs(L):
    if getattr(L, "_wire_sigs", False):
        return
    c = ctypes
    L.phobos_segment_decode.restype, L.phobos_segment_decode.argtypes = c.c_void_p, [c.c_char_p, c.c_size_t]
    L.phobos_segment_free.restype, L.phobos_segment_free.argtypes = None, [c.c_void_p]
    L.phobos_segment_id.restype, L.phobos_segment_id.argtypes = c.c_uint64, [c.c_void_p]
    L.phobos_segment_n_instrs.restype, L.phobos_segment_n_instrs.argtypes = c.c_int32, [c.c_void_p]
    L.phobos_segment_instrs.restype, L.phobos_segment_instrs.argtypes = c.c_void_p, [c.c_void_p]
    L.phobos_segment_encode.restype = c.c_size_t
    L.phobos_segment_encode.argtypes = [c.c_uint64, c.c_void_p, c.c_int32, c.c_void_p, c.c_size_t]
    L._wire_sigs = True


def _instrs_from_array(ptr, n):
    from . import PhInstr
    from .executor import Instr
    arr = ctypes.cast(ptr, ctypes.POINTER(PhInstr)) if ptr else None
    out = []
    for i in range(n):
        a = arr[i]
        out.append(Instr(
            iid=int(a.iid), op=int(a.op), deps=tuple(int(a.deps[d]) for d in range(a.n_deps)), tile=int(a.tile),
            data_type=int(a.data_type), shape=tuple(int(a.shape[d]) for d in range(a.shape_rank)), tensor=int(a.tensor),
            region_offset=tuple(int(a.region.offset[d]) for d in range(a.region.rank)),
            region_shape=tuple(int(a.region.shape[d]) for d in range(a.region.rank)), from_node=int(a.from_node),
            kernel=int(a.kernel), args=tuple((int(a.args[j].tile), int(a.args[j].mode)) for j in range(a.n_args)),
            scalars=tuple(_copy_scalar(a.scalars[j]) for j in range(a.n_scalars)),
            grid=tuple(int(a.grid[d]) for d in range(3)), cta=tuple(int(a.cta[d]) for d in range(3)),
            expected_serves=int(a.expected_serves)))
    return out


def decode_segment(data: bytes):
    """bytes of a phobos.v1.Segment -> (segment id, [Instr, ...])."""
    from . import PH_ERR_PARSE, PhobosError, last_error, lib
    L = lib()
    _wire_sigs(L)
    h = L.phobos_segment_decode(data, len(data))
    if not h:
        raise PhobosError(PH_ERR_PARSE, last_error())
    try:
        return int(L.phobos_segment_id(h)), _instrs_from_array(L.phobos_segment_instrs(h), L.phobos_segment_n_instrs(h))
    finally:
        L.phobos_segment_free(h)


def encode_segment(seg_id: int, instrs) -> bytes:
    """(segment id, [Instr, ...]) -> bytes of a phobos.v1.Segment."""
    from . import PH_ERR_INVALID, PhobosError, last_error, lib
    from .executor import instr_array
    L = lib()
    _wire_sigs(L)
    arr, keep = instr_array(list(instrs))
    n = L.phobos_segment_encode(seg_id, arr, len(keep[0]), None, 0)
    if n == ctypes.c_size_t(-1).value:
        raise PhobosError(PH_ERR_INVALID, last_error())
    buf = ctypes.create_string_buffer(max(1, n))
    L.phobos_segment_encode(seg_id, arr, len(keep[0]), buf, n)
    return buf.raw[:n]
