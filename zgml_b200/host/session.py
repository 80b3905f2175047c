"""Serving session over compiled device programs: the step function every sequence model of the framework is driven by.

A model object provides
  * `vocab`                       — logits per position,
  * `state_specs(max_chunk, max_context)` — the per-sequence device state it carries between steps (host/state.py); a model
                                    that caches every position (`bounded_context`) sizes its caches for `max_context`
                                    positions, and the session refuses to advance a sequence past them,
  * `lower(T, head, pool)`        — the DeviceProgram that advances one sequence by exactly T tokens from the pool's
                                    state (`head` = "none" | "last" | "all": which positions' logits it produces).

`SequenceSession.feed(request, tokens, want)` cuts the request's next tokens into chunks from a fixed menu of program
sizes (powers of two up to `max_chunk`, compiled on first use and kept), writes the control buffer (position, state slot,
token ids) and executes; the CUDA graph of a program is replayed unchanged from step to step.  How a prompt is cut
changes nothing but rounding: state is carried exactly, and every chunk attends through the same key ring.
`step(entries, end)` is the batch form (requests are advanced one after the other, each alone in its program, so a
request's logits cannot depend on its neighbours); `generate` is greedy / sampled decoding on top of `feed`.
"""
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .. import abi
from ..backend import CudaBackend, DeviceProgram, ProgramIO
from .sampling import Sampler
from .state import SequenceStatePool


@dataclass
class LoweredProgram:
    program: DeviceProgram
    buf_ctl: int
    buf_logits: Optional[int]      # None for head == "none"
    logits_rows: int
    layer_bufs: Optional[List[int]] = None   # residual stream after every layer (debug lowering only)


def chunk_menu(max_chunk: int) -> List[int]:
    m, out = 1, []
    while m <= max_chunk:
        out.append(m)
        m *= 2
    return out[::-1]


def cut(n: int, menu: Sequence[int]) -> List[int]:
    """Greedy decomposition of n tokens into menu sizes, largest first."""
    out = []
    for m in menu:
        while n >= m:
            out.append(m)
            n -= m
    assert n == 0
    return out


class SequenceSession:
    def __init__(self, be: CudaBackend, model, n_slots: int = 1, max_chunk: int = 256, keep_layers: bool = False,
                 max_context: Optional[int] = None):
        self.be, self.model, self.keep_layers = be, model, keep_layers
        self.menu = chunk_menu(max_chunk)
        self.max_chunk = self.menu[0]
        self.pool = SequenceStatePool(be, model.state_specs(self.max_chunk, max_context), n_slots)
        self.context_limit = model.capacity(self.max_chunk, max_context) if getattr(model, "bounded_context", False) else None
        self._programs: Dict[Tuple[int, str], tuple] = {}
        self.executions = 0

    # ── programs ──
    def program(self, T: int, head: str):
        key = (T, head)
        if key not in self._programs:
            lp = self.model.lower(T, head, self.pool, keep_layers=self.keep_layers)
            handle = self.be.compile_program(lp.program)
            if handle is None:
                from ..backend import last_error
                raise RuntimeError(f"compile_program failed for T = {T}, head = {head}: {last_error()}")
            ctl = np.zeros(abi.CTL_IDS + T, np.int32)
            logits = np.zeros((lp.logits_rows, self.model.vocab), np.float32) if lp.buf_logits is not None else None
            self._programs[key] = (lp, handle, ctl, logits)
        return self._programs[key]

    def _run(self, T, head, slot, pos, tokens):
        lp, handle, ctl, logits = self.program(T, head)
        ctl[abi.CTL_POS], ctl[abi.CTL_SLOT] = pos, slot
        ctl[abi.CTL_IDS:] = tokens
        outs = [ProgramIO(lp.buf_logits, logits)] if logits is not None else []
        self.be.execute_program(handle, [ProgramIO(lp.buf_ctl, ctl)], outs)
        self.executions += 1
        return logits

    # ── the step function ──
    def feed(self, request_id, tokens: Sequence[int], want: Iterable[int] = ()) -> np.ndarray:
        """Advance `request_id` by `tokens`; returns the logits at the places `want` (indices into `tokens`), in order."""
        tokens = [int(t) for t in tokens]
        if any(t < 0 or t >= self.model.vocab for t in tokens):
            raise ValueError("token id outside the vocabulary")
        want = [int(w) for w in want]
        if any(w < 0 or w >= len(tokens) for w in want):
            raise ValueError("wanted place outside the step's tokens")
        slot = self.pool.acquire(request_id)
        if self.context_limit is not None and self.pool.position(request_id) + len(tokens) > self.context_limit:
            raise ValueError(f"request {request_id!r} would reach position {self.pool.position(request_id) + len(tokens)}: the session's caches hold "
                             f"{self.context_limit} positions per sequence")
        rows: Dict[int, np.ndarray] = {}
        at = 0
        for T in cut(len(tokens), self.menu):
            local = sorted({w - at for w in want if at <= w < at + T})
            head = "none" if not local else ("last" if local == [T - 1] else "all")
            logits = self._run(T, head, slot, self.pool.position(request_id), tokens[at:at + T])
            for w in local:
                rows[at + w] = logits[0 if head == "last" else w].copy()
            self.pool.advance(request_id, T)
            at += T
        return np.stack([rows[w] for w in want]) if want else np.zeros((0, self.model.vocab), np.float32)

    def release(self, request_id):
        self.pool.release(request_id)

    def step(self, entries: Sequence[dict], end: Iterable = ()) -> List[np.ndarray]:
        """entries: [{"id", "tokens", "want"}]; `end`: requests whose state is given back after the step."""
        out = [self.feed(e["id"], e["tokens"], e.get("want", ())) for e in entries]
        for r in end:
            self.release(r)
        return out

    def layer_streams(self, T: int, head: str) -> np.ndarray:
        """Residual stream after every layer of the last execution of program (T, head); needs keep_layers."""
        lp, handle, _, _ = self._programs[(T, head)]
        assert lp.layer_bufs is not None
        width = self.model.width
        out = np.zeros((len(lp.layer_bufs), T, width), np.float32)
        for i, b in enumerate(lp.layer_bufs):
            self.be.read_buffer(handle, b, out[i])
        return out

    def generate(self, prompt: Sequence[int], max_new_tokens: int, sampler: Optional[Sampler] = None, request_id="generate",
                 stop: Optional[int] = None) -> List[int]:
        """Prefill `prompt`, then decode token by token through the same step function."""
        sampler = sampler or Sampler()
        logits = self.feed(request_id, prompt, [len(prompt) - 1])[0]
        out: List[int] = []
        try:
            for _ in range(max_new_tokens):
                tok = sampler(logits)
                out.append(tok)
                if stop is not None and tok == stop:
                    break
                if len(out) < max_new_tokens:
                    logits = self.feed(request_id, [tok], [0])[0]
        finally:
            self.release(request_id)
        return out

    def close(self):
        for _, handle, _, _ in self._programs.values():
            self.be.free_program(handle)
        self._programs = {}
        self.pool.close()
