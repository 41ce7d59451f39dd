"""Cooked world template container (".nkt").

One env's template (the role of the reference's cooked ``nk::Model``,
src/nk/model/model.hpp:175-244) as a flat list of named arrays:

    "NKT1" | u32 count | { char name[32] | u32 dtype | u32 pad | u64 n | data padded to 8 bytes }

dtype: 0 float32, 1 uint32, 2 int32, 3 uint64.  The native library parses this blob in
``nuka_world_create_from_template``; ``scene_path`` values ending in ".nkt" load it from disk.
"""
import struct

import numpy as np

_DTYPES = {np.dtype(np.float32): 0, np.dtype(np.uint32): 1, np.dtype(np.int32): 2, np.dtype(np.uint64): 3}
_FROM = {0: np.float32, 1: np.uint32, 2: np.int32, 3: np.uint64}


def pack(arrays):
    """Serialise a dict name -> ndarray into template bytes."""
    out = [b"NKT1", struct.pack("<I", len(arrays))]
    for name, value in arrays.items():
        a = np.ascontiguousarray(value)
        if a.dtype not in _DTYPES:
            raise TypeError(f"template field {name}: unsupported dtype {a.dtype}")
        raw = a.tobytes()
        nm = name.encode()
        if len(nm) > 31:
            raise ValueError(f"template field name too long: {name}")
        out.append(nm.ljust(32, b"\0"))
        out.append(struct.pack("<IIQ", _DTYPES[a.dtype], 0, a.size))
        out.append(raw + b"\0" * (-len(raw) % 8))
    return b"".join(out)


def unpack(blob):
    """Inverse of :func:`pack`."""
    if blob[:4] != b"NKT1":
        raise ValueError("not a template blob")
    (count,) = struct.unpack_from("<I", blob, 4)
    at, arrays = 8, {}
    for _ in range(count):
        name = blob[at:at + 32].split(b"\0", 1)[0].decode()
        dtype, _, n = struct.unpack_from("<IIQ", blob, at + 32)
        dt = np.dtype(_FROM[dtype])
        nbytes = n * dt.itemsize
        arrays[name] = np.frombuffer(blob, dtype=dt, count=n, offset=at + 48).copy()
        at += 48 + nbytes + (-nbytes % 8)
    return arrays
