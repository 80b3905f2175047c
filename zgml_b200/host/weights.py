"""Device-resident weights of the sequence models: tensors packed back to back in one buffer per layer, in the session's
weight format (bfloat16 bit patterns or f32), addressed by element offset from the lowering."""
from typing import Dict, List

import numpy as np

from .. import abi
from ..backend import CudaBackend, DeviceBuffer
from .safetensors import f32_to_bf16_bits


class WeightArena:
    """Tensors of one layer packed back to back (16-byte aligned starts) in the session's weight format."""

    def __init__(self, wdt: int):
        self.wdt = wdt
        self.parts: List[np.ndarray] = []
        self.off: Dict[str, int] = {}
        self.n = 0

    def add(self, name: str, a: np.ndarray) -> int:
        a = np.ascontiguousarray(a, dtype=np.float32).ravel()
        pad = -self.n % 8
        if pad:
            self.parts.append(np.zeros(pad, np.float32))
            self.n += pad
        self.off[name] = self.n
        self.parts.append(a)
        self.n += a.size
        return self.off[name]

    def upload(self, be: CudaBackend) -> DeviceBuffer:
        flat = np.concatenate(self.parts) if self.parts else np.zeros(8, np.float32)
        host = f32_to_bf16_bits(flat) if self.wdt == abi.W_BF16 else flat     # checkpoint values are bfloat16: exact either way
        buf = DeviceBuffer(be, host.nbytes, zero=False)
        buf.upload(host)
        self.parts = []
        return buf
