"""Tiny named-array container shared by the reference-kernel harness (C++) and the tests (Python).

TEST INFRASTRUCTURE ONLY - nothing in the product path reads or writes this format.

File layout (little endian):
    magic   4 bytes  b"MSCB"
    count   u32      number of entries
    entry*  char name[48] (NUL padded) | u32 dtype | u32 reserved | u64 n_elements | data, padded to 8 bytes

dtype codes: 0 f32, 1 u32, 2 i32, 3 u16, 4 u8, 5 f64
"""
import struct

import numpy as np

_DTYPES = {0: np.float32, 1: np.uint32, 2: np.int32, 3: np.uint16, 4: np.uint8, 5: np.float64}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


def write_bundle(path, arrays):
    """arrays: dict name -> 1-D (or any shape; flattened) numpy array of a supported dtype."""
    with open(path, "wb") as f:
        f.write(b"MSCB")
        f.write(struct.pack("<I", len(arrays)))
        for name, arr in arrays.items():
            a = np.ascontiguousarray(arr).reshape(-1)
            code = _CODES[a.dtype]
            nm = name.encode()
            assert len(nm) < 48, name
            f.write(nm + b"\0" * (48 - len(nm)))
            f.write(struct.pack("<IIQ", code, 0, a.size))
            raw = a.tobytes()
            f.write(raw)
            f.write(b"\0" * ((-len(raw)) % 8))


def read_bundle(path):
    out = {}
    with open(path, "rb") as f:
        assert f.read(4) == b"MSCB", "not a bundle file"
        (count,) = struct.unpack("<I", f.read(4))
        for _ in range(count):
            name = f.read(48).split(b"\0", 1)[0].decode()
            code, _, n = struct.unpack("<IIQ", f.read(16))
            dt = np.dtype(_DTYPES[code])
            nbytes = n * dt.itemsize
            data = f.read(nbytes)
            f.read((-nbytes) % 8)
            out[name] = np.frombuffer(data, dtype=dt).copy()
    return out
