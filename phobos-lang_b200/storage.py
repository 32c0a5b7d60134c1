"""file:// tensor storage: headerless row-major blobs with region LOAD / STORE
(phobos-cluster/src/storage.rs:9-79)."""
from __future__ import annotations

import ctypes

import numpy as np

_NP = {0: np.float16, 1: np.float32, 2: np.float64, 3: np.int8, 4: np.int32, 5: np.int64, 6: np.bool_}


def storage_path(uri: str) -> str:
    from . import check, lib
    buf = ctypes.create_string_buffer(4096)
    check(lib().phobos_storage_path(uri.encode(), buf, 4096))
    return buf.value.decode()


def _region(offset, shape):
    from . import PhRegion
    r = PhRegion()
    r.rank = len(shape)
    for i, (o, s) in enumerate(zip(offset, shape)):
        r.offset[i], r.shape[i] = o, s
    return r


def load_region(uri: str, tensor_shape, offset, shape, dtype: int = 1) -> np.ndarray:
    """Gathers the region's row spans into a contiguous array (storage.rs:48-60)."""
    from . import check, lib
    out = np.empty(tuple(shape), dtype=_NP[dtype])
    ts = (ctypes.c_uint64 * len(tensor_shape))(*tensor_shape)
    reg = _region(offset, shape)
    check(lib().phobos_storage_load(uri.encode(), ts, len(tensor_shape), ctypes.byref(reg), out.itemsize,
                                    out.ctypes.data_as(ctypes.c_void_p)))
    return out


def store_region(uri: str, tensor_shape, offset, data: np.ndarray) -> None:
    """Scatters a contiguous tile back into the file without truncating it (storage.rs:62-79)."""
    from . import check, lib
    data = np.ascontiguousarray(data)
    ts = (ctypes.c_uint64 * len(tensor_shape))(*tensor_shape)
    reg = _region(offset, data.shape)
    check(lib().phobos_storage_store(uri.encode(), ts, len(tensor_shape), ctypes.byref(reg), data.itemsize,
                                     data.ctypes.data_as(ctypes.c_void_p)))
