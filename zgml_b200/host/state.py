"""Per-sequence device state shared by the compiled programs of one serving session.

A model's lowering names the state it carries from step to step as `StateSpec`s (a key ring of a windowed attention
layer, the matrix state of a recurrent layer, the input tail of a short convolution).  `SequenceStatePool` allocates
each as ONE device buffer `[slots, per-slot elements]` (f32), hands out slots to requests, remembers every request's
position and gives a slot back — zeroed where the spec asks for it — when the request ends.  Programs reference the
buffers as external buffers and pick the slot through their control buffer, so any program of the session can continue
any live sequence.
"""
from dataclasses import dataclass
from typing import Dict, List

from ..backend import CudaBackend, DeviceBuffer


@dataclass(frozen=True)
class StateSpec:
    name: str
    elems: int            # f32 elements per slot
    zero_on_acquire: bool  # recurrent state and convolution tails start at zero; a key ring is masked by position instead


class SequenceStatePool:
    def __init__(self, be: CudaBackend, specs: List[StateSpec], n_slots: int = 1):
        assert n_slots >= 1
        self.be, self.specs, self.n_slots = be, list(specs), n_slots
        self.buffers: Dict[str, DeviceBuffer] = {s.name: DeviceBuffer(be, 4 * s.elems * n_slots) for s in self.specs}
        self._free = list(range(n_slots - 1, -1, -1))
        self._slot: Dict[str, int] = {}
        self._pos: Dict[str, int] = {}

    # ── slots ──
    def live(self):
        return list(self._slot)

    def has(self, request_id) -> bool:
        return request_id in self._slot

    def acquire(self, request_id) -> int:
        if request_id in self._slot:
            return self._slot[request_id]
        if not self._free:
            raise RuntimeError(f"no free state slot for request {request_id!r} ({self.n_slots} live)")
        slot = self._free.pop()
        for s in self.specs:   # a reused slot must not leak the previous sequence's state
            if s.zero_on_acquire:
                self.buffers[s.name].fill_zero(4 * s.elems * slot, 4 * s.elems)
        self._slot[request_id], self._pos[request_id] = slot, 0
        return slot

    def release(self, request_id):
        slot = self._slot.pop(request_id, None)
        self._pos.pop(request_id, None)
        if slot is not None:
            self._free.append(slot)

    def slot(self, request_id) -> int:
        return self._slot[request_id]

    def position(self, request_id) -> int:
        return self._pos[request_id]

    def advance(self, request_id, n: int):
        self._pos[request_id] += n

    def bytes(self) -> int:
        return sum(b.nbytes for b in self.buffers.values())

    def close(self):
        for b in self.buffers.values():
            b.free()
        self.buffers = {}
