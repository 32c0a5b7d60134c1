"""Instruction executor front end: ALLOC / LOAD / FETCH / COMPUTE / STORE / FREE with
dependency lists, as the pod's Engine runs them (phobos-pod/src/engine.rs:282-398)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field


@dataclass
class Instr:
    """One instruction (phobos-cluster/src/isa.rs:24-58).  Only the fields of its op are read."""
    iid: int
    op: int
    deps: tuple = ()
    tile: int = 0
    data_type: int = 1
    shape: tuple = ()
    tensor: int = 0
    region_offset: tuple = ()
    region_shape: tuple = ()
    from_node: int = 0
    kernel: int = 0
    args: tuple = ()        # ((tile, mode), ...)
    scalars: tuple = ()     # PhScalar, ...
    grid: tuple = (1, 1, 1)
    cta: tuple = (256, 1, 1)
    expected_serves: int = 0
    _keep: list = field(default_factory=list, repr=False)


def device_uri(t) -> str:
    """Storage URI of a contiguous CUDA tensor that stays alive for the job: `device://<gpu>/0x<address>`.  A job
    whose tensors carry such URIs keeps them in HBM: LOAD and STORE become 2-D device copies (over NVLink from
    another GPU) instead of file reads through pinned host memory."""
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("device_uri needs a contiguous CUDA tensor")
    return f"device://{t.device.index}/0x{t.data_ptr():x}"


def instr_array(instrs):
    """[Instr, ...] -> (ctypes array of PhInstr, objects that must stay alive while the array is used)."""
    from . import PhInstr, PhScalar, PhTileArg
    arr = (PhInstr * max(1, len(instrs)))()
    keep = [instrs]
    for i, ins in enumerate(instrs):
        a = arr[i]
        a.iid, a.op, a.tile = ins.iid, ins.op, ins.tile
        deps = (ctypes.c_uint64 * max(1, len(ins.deps)))(*ins.deps)
        keep.append(deps)
        a.deps, a.n_deps = deps, len(ins.deps)
        a.data_type, a.shape_rank = ins.data_type, len(ins.shape)
        for d, s in enumerate(ins.shape):
            a.shape[d] = s
        a.tensor = ins.tensor
        a.region.rank = len(ins.region_shape)
        for d, (o, s) in enumerate(zip(ins.region_offset, ins.region_shape)):
            a.region.offset[d], a.region.shape[d] = o, s
        a.from_node, a.kernel = ins.from_node, ins.kernel
        args = (PhTileArg * max(1, len(ins.args)))(*[PhTileArg(t, m) for t, m in ins.args])
        keep.append(args)
        a.args, a.n_args = args, len(ins.args)
        sc = (PhScalar * max(1, len(ins.scalars)))(*ins.scalars)
        keep.append(sc)
        a.scalars, a.n_scalars = sc, len(ins.scalars)
        for d in range(3):
            a.grid[d], a.cta[d] = ins.grid[d], ins.cta[d]
        a.expected_serves = ins.expected_serves
    return arr, keep


class Executor:
    def __init__(self, device: int = 0, node_id: int = 0, arena_bytes: int = 512 << 20):
        from . import PH_ERR_DEVICE, PhobosError, last_error, lib
        self._L = lib()
        self._h = self._L.phobos_executor_create(device, node_id, arena_bytes)
        if not self._h:
            raise PhobosError(PH_ERR_DEVICE, last_error())
        self.node_id = node_id
        self._uris = []

    def close(self) -> None:
        if self._h:
            self._L.phobos_executor_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_tensors(self, tensors) -> None:
        """tensors: iterable of (uri, dtype, shape, mode) — EngineMsg::SetTensors."""
        from . import PhTensorMeta, check
        tensors = list(tensors)
        arr = (PhTensorMeta * max(1, len(tensors)))()
        self._uris = [t[0].encode() for t in tensors]
        for i, (uri, dtype, shape, mode) in enumerate(tensors):
            arr[i].uri = self._uris[i]
            arr[i].dtype = dtype
            arr[i].rank = len(shape)
            for d, s in enumerate(shape):
                arr[i].shape[d] = s
            arr[i].mode = mode
        check(self._L.phobos_executor_set_tensors(self._h, arr, len(tensors)))

    def set_kernel(self, kernel_id: int, entry: str, kind_hint: int = -1) -> None:
        from . import check
        check(self._L.phobos_executor_set_kernel(self._h, kernel_id, entry.encode(), kind_hint))

    def connect_peer(self, node_id: int, peer: "Executor") -> None:
        from . import check
        check(self._L.phobos_executor_connect_peer(self._h, node_id, peer._h))

    def issue(self, instrs) -> None:
        """EngineMsg::Issue(Segment): adds the instructions and wires their dependency counters."""
        from . import check
        arr, keep = instr_array(list(instrs))
        check(self._L.phobos_executor_issue(self._h, arr, len(keep[0])))

    def run(self) -> None:
        """Runs until nothing is pending; raises on the first failed instruction."""
        from . import check
        check(self._L.phobos_executor_run(self._h))

    def completions(self):
        from . import PhCompletion
        buf = (PhCompletion * 256)()
        out = []
        while True:
            n = self._L.phobos_executor_drain_completions(self._h, buf, 256)
            out.extend((int(buf[i].iid), int(buf[i].status), int(buf[i].elapsed_ns)) for i in range(n))
            if n < 256:
                return out

    @property
    def last_run_ms(self) -> float:
        """Device time (CUDA events) of the last run, from its start to its last operation; -1 before any run."""
        return float(self._L.phobos_executor_last_run_ms(self._h))

    @property
    def arena_used(self) -> int:
        return int(self._L.phobos_executor_arena_used(self._h))

    @property
    def served_bytes(self) -> int:
        return int(self._L.phobos_executor_served_bytes(self._h))

    def tile_addr(self, tile: int):
        from . import check
        addr = ctypes.c_void_p()
        res = ctypes.c_int32()
        check(self._L.phobos_executor_tile_addr(self._h, tile, ctypes.byref(addr), ctypes.byref(res)))
        return addr.value, bool(res.value)
