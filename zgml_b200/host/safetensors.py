"""Reader / writer of the safetensors container: an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets relative to the end of the header) and the raw tensor data.

The file is memory-mapped; `raw(name)` hands out views without copying.  bfloat16 has no numpy dtype: such
tensors are exposed as uint16 bit patterns (`bf16_bits`) or widened exactly to float32 (`f32`).
"""
import json
import mmap
import struct
from typing import Dict, Tuple

import numpy as np

_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I32": np.int32, "I64": np.int64, "U8": np.uint8, "I8": np.int8,
       "F64": np.float64}


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even narrowing (NaN payloads are not preserved)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


class SafetensorsFile:
    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._mm[:8])
        if n > len(self._mm) - 8:
            raise ValueError(f"{path}: header length {n} exceeds the file")
        header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self.entries: Dict[str, Tuple[str, tuple, int, int]] = {}
        for name, e in header.items():
            lo, hi = e["data_offsets"]
            if e["dtype"] not in _NP:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
            if hi < lo or self._base + hi > len(self._mm):
                raise ValueError(f"{path}: tensor {name} lies outside the file")
            self.entries[name] = (e["dtype"], tuple(e["shape"]), lo, hi)

    def names(self):
        return list(self.entries)

    def __contains__(self, name):
        return name in self.entries

    def shape(self, name) -> tuple:
        return self.entries[name][1]

    def dtype(self, name) -> str:
        return self.entries[name][0]

    def raw(self, name) -> np.ndarray:
        dt, shape, lo, hi = self.entries[name]
        a = np.frombuffer(self._mm, dtype=_NP[dt], count=(hi - lo) // np.dtype(_NP[dt]).itemsize, offset=self._base + lo)
        return a.reshape(shape)

    def f32(self, name) -> np.ndarray:
        dt = self.entries[name][0]
        a = self.raw(name)
        return bf16_bits_to_f32(a) if dt == "BF16" else a.astype(np.float32)

    def bf16_bits(self, name) -> np.ndarray:
        dt = self.entries[name][0]
        a = self.raw(name)
        return a if dt == "BF16" else f32_to_bf16_bits(a.astype(np.float32))

    def close(self):
        try:
            self._mm.close()
        except BufferError:      # views handed out by raw() are still alive; the map goes with them
            pass
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], bf16: bool = True):
    """Test / tooling helper: float arrays are stored as bfloat16 (rounded) when `bf16`, integer arrays as int32."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.asarray(a)
        if np.issubdtype(a.dtype, np.integer):
            dt, blob = "I32", np.ascontiguousarray(a, dtype="<i4").tobytes()
        elif bf16:
            dt, blob = "BF16", f32_to_bf16_bits(a.astype(np.float32)).astype("<u2").tobytes()
        else:
            dt, blob = "F32", np.ascontiguousarray(a, dtype="<f4").tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(blob)]}
        blobs.append(blob)
        off += len(blob)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
