"""Job-file binding: `source = / dim / tensor / scalar` (phobos-sched/src/job.rs:5-88)."""
from __future__ import annotations

import struct
from dataclasses import dataclass, field


@dataclass
class JobTensor:
    name: str
    dtype: int
    mode: int
    shape: tuple
    uri: str


@dataclass
class JobScalar:
    name: str
    dtype: int
    bits: int

    @property
    def value(self):
        from . import BOOL, F32, F64, I32, I64
        if self.dtype == F32:
            return struct.unpack("<f", struct.pack("<I", self.bits & 0xFFFFFFFF))[0]
        if self.dtype == F64:
            return struct.unpack("<d", struct.pack("<Q", self.bits))[0]
        if self.dtype == I32:
            return struct.unpack("<i", struct.pack("<I", self.bits & 0xFFFFFFFF))[0]
        if self.dtype == I64:
            return struct.unpack("<q", struct.pack("<Q", self.bits))[0]
        if self.dtype == BOOL:
            return bool(self.bits)
        raise ValueError(self.dtype)


@dataclass
class Job:
    kernel: str
    dims: dict = field(default_factory=dict)
    tensors: list = field(default_factory=list)
    scalars: list = field(default_factory=list)
    source: str = ""                    # text of the `source =` file
    _handle: object = field(default=None, repr=False, compare=False)

    def __del__(self):
        if self._handle:
            from . import lib
            lib().phobos_job_free(self._handle)
            self._handle = None


def _collect(handle) -> Job:
    from . import lib
    L = lib()
    try:
        job = Job(kernel=L.phobos_job_kernel_name(handle).decode())
        for i in range(L.phobos_job_n_dims(handle)):
            job.dims[L.phobos_job_dim_name(handle, i).decode()] = int(L.phobos_job_dim_value(handle, i))
        for i in range(L.phobos_job_n_tensors(handle)):
            rank = L.phobos_job_tensor_rank(handle, i)
            job.tensors.append(JobTensor(
                name=L.phobos_job_tensor_name(handle, i).decode(), dtype=int(L.phobos_job_tensor_dtype(handle, i)),
                mode=int(L.phobos_job_tensor_mode(handle, i)),
                shape=tuple(int(L.phobos_job_tensor_dim(handle, i, d)) for d in range(rank)),
                uri=L.phobos_job_tensor_uri(handle, i).decode()))
        for i in range(L.phobos_job_n_scalars(handle)):
            job.scalars.append(JobScalar(name=L.phobos_job_scalar_name(handle, i).decode(),
                                         dtype=int(L.phobos_job_scalar_dtype(handle, i)),
                                         bits=int(L.phobos_job_scalar_bits(handle, i))))
        job.source = L.phobos_job_source(handle).decode()
        job._handle = handle
        return job
    except Exception:
        L.phobos_job_free(handle)
        raise


def parse_job(path: str) -> Job:
    """Reads a job file; raises PhobosError with `path:line: message` as the reference does."""
    from . import PH_ERR_PARSE, PhobosError, last_error, lib
    h = lib().phobos_job_parse(str(path).encode())
    if not h:
        raise PhobosError(PH_ERR_PARSE, last_error())
    return _collect(h)


def parse_job_text(text: str, origin: str = "<text>", source_text: str | None = None) -> Job:
    """As parse_job, from a string; `source_text` stands in for the file the `source =` line names."""
    from . import PH_ERR_PARSE, PhobosError, last_error, lib
    h = lib().phobos_job_parse_text(text.encode(), origin.encode(),
                                    None if source_text is None else source_text.encode())
    if not h:
        raise PhobosError(PH_ERR_PARSE, last_error())
    return _collect(h)
