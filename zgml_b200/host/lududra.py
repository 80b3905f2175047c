"""Lududra: a decoder-only stack whose layers pair a token mixer — sliding-window attention with a sink, or a gated
delta-rule recurrence with per-channel decay — with an optional routed mixture of experts, each sublayer between a
layer norm before and a layer norm after it.

This file is the model's configuration reader, its weight packer and its LOWERING to a DeviceProgram; all arithmetic
happens in the sequence-model DeviceOps of the CUDA library (csrc/seqops.cu) and all state in the session's
`SequenceStatePool`.  Every size and every per-model constant comes from config.json or a tensor's shape.

Per layer (x: residual stream, f32):
    h = LN(x; norm1);  y = mixer(h);  x = x + LN(y; norm1b);  h = LN(x; norm2);  y = moe(h);  x = x + LN(y; norm2b)

attention mixer   [q | k | gate] = W_in h + b in ONE matmul (the checkpoint's q, k, g stacked at load; the keys are also
                  the values), then the WINDOW_ATTENTION op: window, smooth score cap, per-distance bias (the learned
                  bucket table expanded to one row per distance at load), sink, output gate; then W_o.
channel_delta     [q | k | v | beta | a1 | g1] = W_in h in ONE matmul, one CAUSAL_CONV (+SiLU) over the q | k | v
                  columns, the two low-rank second stages (decay and gate) as one block-diagonal matmul, the DELTA_RULE op, then W_o.
moe               router matmul (f32 activations), ROUTE (softmax over real and identity experts, top-k of the corrected
                  scores, uncorrected weights), MOE_FFN over stacked expert weights.
"""
import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import abi
from ..backend import CudaBackend, DeviceBuffer, DeviceOp, DeviceProgram, ExternBuffer, ProgramIO, seq_scratch_elems
from .safetensors import SafetensorsFile
from .session import LoweredProgram
from .state import SequenceStatePool, StateSpec
from .weights import WeightArena as _Arena

ARCHITECTURE = "Lududra"
UNIT_EPS = 1e-6          # inside the root of the q / k unit vectors
EXPERT_ALPHA = 1.702     # g * sigmoid(alpha * g)


@dataclass(frozen=True)
class LududraConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple            # of dicts: {"type", "mixer": {...}, "mlp": {...} | None}

    @classmethod
    def from_dict(cls, c: dict) -> "LududraConfig":
        if c.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture = {c.get('architecture')!r}")
        layers = []
        for i, L in enumerate(c["layers"]):
            m = L["mixer"]
            if L["type"] == "attention":
                if m["vdim"] != m["dim"]:
                    raise ValueError(f"layer {i}: keys double as values, so vdim must equal dim")
                if m["heads"] % m["kv_heads"]:
                    raise ValueError(f"layer {i}: heads not a multiple of kv_heads")
            elif L["type"] == "channel_delta":
                if m["heads"] % m["kv_heads"]:
                    raise ValueError(f"layer {i}: heads not a multiple of kv_heads")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append({"type": L["type"], "mixer": dict(m), "mlp": mlp})
        return cls(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), float(c["embedding"]["scale"]), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "LududraConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


def distance_bucket(n: int, n_rows: int, bias_max: float) -> int:
    """Row of the learned distance-bias table for distance n: one row per distance below n_rows / 2, then
    logarithmically spaced rows that reach the last one at distance bias_max."""
    half = n_rows // 2
    if n < half:
        return n
    return min(n_rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (n_rows - half))))


def distance_bias_table(rel: np.ndarray, window: int, bias_max: float) -> np.ndarray:
    """[window, heads] f32: the bias of every distance the window can see (what WINDOW_ATTENTION indexes)."""
    rows = [distance_bucket(n, rel.shape[0], bias_max) for n in range(window)]
    return np.ascontiguousarray(rel[rows], dtype=np.float32)


class LududraModel:
    """Weights resident in HBM (one arena per layer + one for embedding / final norm / head) and the lowering."""

    def __init__(self, be: CudaBackend, cfg: LududraConfig, tensors, dtype: str = "bfloat16"):
        """tensors: name -> f32 array accessor (`tensors(name)`), e.g. SafetensorsFile.f32."""
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.be, self.cfg, self.dtype = be, cfg, dtype
        self.wdt = abi.W_BF16 if dtype == "bfloat16" else abi.W_F32
        self.vocab, self.width = cfg.vocab, cfg.width
        self.layer_meta: List[dict] = []
        self.arenas: List[_Arena] = []
        self.buffers: List[DeviceBuffer] = []
        self.bias_tables: List[Optional[np.ndarray]] = []
        D = cfg.width
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L["mixer"]
            A = _Arena(self.wdt)
            meta = {"type": L["type"]}
            A.add("norm1", tensors(p + "norm1"))
            A.add("norm1b", tensors(p + "norm1b"))
            H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            if L["type"] == "attention":
                q, k, g = tensors(p + "mix.q"), tensors(p + "mix.k"), tensors(p + "mix.g")
                assert q.shape == (H * dim, D) and k.shape == (G * dim, D) and g.shape == (H * vdim, D)
                A.add("in", np.concatenate([q, k, g], 0))
                A.add("in.b", np.concatenate([tensors(p + "mix.q.b"), tensors(p + "mix.k.b"), np.zeros(H * vdim, np.float32)]))
                meta.update(n_in=H * dim + G * dim + H * vdim, q_off=0, k_off=H * dim, g_off=H * dim + G * dim)
                self.bias_tables.append(distance_bias_table(tensors(p + "mix.rel"), m["mask"]["size"], m["bias_max"]))
            else:
                q, k, v = tensors(p + "mix.q"), tensors(p + "mix.k"), tensors(p + "mix.v")
                b, a1, g1 = tensors(p + "mix.b"), tensors(p + "mix.a1"), tensors(p + "mix.g1")
                assert q.shape == (G * dim, D) and k.shape == (G * dim, D) and v.shape == (H * vdim, D) and b.shape == (H, D)
                C = 2 * G * dim + H * vdim
                ra, rg = a1.shape[0], g1.shape[0]
                A.add("in", np.concatenate([q, k, v, b, a1, g1], 0))
                convs = [tensors(p + f"mix.{n}.conv") for n in "qkv"]
                taps = convs[0].shape[1]
                assert all(c.shape[1] == taps for c in convs) and taps == m["conv"]
                A.add("conv", np.concatenate(convs, 0))
                a2, g2 = tensors(p + "mix.a2"), tensors(p + "mix.g2")
                assert a2.shape == (H * dim, ra) and g2.shape == (H * vdim, rg)
                # both low-rank second stages as ONE matmul over the adjacent a1 | g1 columns: [[a2, 0], [0, g2]]
                ag2 = np.zeros((H * dim + H * vdim, ra + rg), np.float32)
                ag2[:H * dim, :ra], ag2[H * dim:, ra:] = a2, g2
                A.add("ag2", ag2)
                A.add("A_log", tensors(p + "mix.A_log"))
                A.add("dt_bias", tensors(p + "mix.dt_bias"))
                A.add("onorm", tensors(p + "mix.norm"))
                meta.update(n_in=C + H + ra + rg, C=C, taps=taps, ra=ra, rg=rg, beta_off=C, a1_off=C + H, g1_off=C + H + ra)
                self.bias_tables.append(None)
            o = tensors(p + "mix.o")
            assert o.shape == (D, H * vdim)
            A.add("o", o)
            mlp = L["mlp"]
            if mlp is not None:
                r = mlp["router"]
                E, I, ff = r["experts"], r.get("identity", 0), mlp["expert"]["ff"]
                A.add("norm2", tensors(p + "norm2"))
                A.add("norm2b", tensors(p + "norm2b"))
                router = tensors(p + "mlp.router")
                assert router.shape == (E + I, D)
                A.add("router", router)
                A.add("correction", tensors(p + "mlp.correction"))
                for part, shape in (("gate", (ff, D)), ("up", (ff, D)), ("down", (D, ff))):
                    stack = [tensors(p + f"mlp.e{e}.{part}") for e in range(E)]
                    assert all(s.shape == shape for s in stack)
                    A.add(part, np.stack(stack) if stack else np.zeros(0, np.float32))
                meta.update(E=E, NE=E + I, ff=ff, top=r["top"], limit=mlp["expert"]["limit"])
            self.layer_meta.append(meta)
            self.arenas.append(A)
            self.buffers.append(A.upload(be))
        A = _Arena(self.wdt)
        emb, head = tensors("embed"), tensors("head")
        assert emb.shape == (cfg.vocab, D) and head.shape == (cfg.vocab, D)
        A.add("embed", emb)
        A.add("final.norm", tensors("final.norm"))
        A.add("head", head)
        self.arenas.append(A)
        self.buffers.append(A.upload(be))

    @classmethod
    def load(cls, be: CudaBackend, model_dir: str, dtype: str = "bfloat16") -> "LududraModel":
        cfg = LududraConfig.from_json(os.path.join(model_dir, "config.json"))
        sf = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
        try:
            return cls(be, cfg, sf.f32, dtype)
        finally:
            sf.close()

    def weight_bytes(self) -> int:
        return sum(b.nbytes for b in self.buffers)

    # ── state ──
    def ring_rows(self, window: int, max_chunk: int) -> int:
        return window - 1 + max_chunk

    def state_specs(self, max_chunk: int, max_context: Optional[int] = None) -> List[StateSpec]:   # state is O(window): no bound on positions
        specs = []
        for i, L in enumerate(self.cfg.layers):
            m = L["mixer"]
            if L["type"] == "attention":
                specs.append(StateSpec(f"l{i}.ring", self.ring_rows(m["mask"]["size"], max_chunk) * m["kv_heads"] * m["dim"], False))
            else:
                C = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
                specs.append(StateSpec(f"l{i}.S", m["heads"] * m["dim"] * m["vdim"], True))
                if m["conv"] > 1:
                    specs.append(StateSpec(f"l{i}.tail", (m["conv"] - 1) * C, True))
        return specs

    # ── lowering ──
    def lower(self, T: int, head: str, pool: SequenceStatePool, keep_layers: bool = False) -> LoweredProgram:
        cfg, wdt, D, eps = self.cfg, self.wdt, self.cfg.width, self.cfg.norm_eps
        sizes: List[int] = []
        uploads: List[ProgramIO] = []
        externs: List[ExternBuffer] = []
        ops = []

        def new(n, init=None):
            sizes.append(max(int(n), 1))
            if init is not None:
                uploads.append(ProgramIO(len(sizes) - 1, np.ascontiguousarray(init, dtype=np.float32).ravel()))
            return len(sizes) - 1

        def ext(buf: DeviceBuffer):
            sizes.append(buf.elems)
            externs.append(ExternBuffer(len(sizes) - 1, buf))
            return len(sizes) - 1

        max_chunk = max(T, 1)
        ctl = new(abi.CTL_IDS + T)
        wbuf = [ext(b) for b in self.buffers]
        gl, GA = wbuf[-1], self.arenas[-1]
        xs = [new(T * D), new(T * D)]
        h, y = new(T * D), new(T * D)
        n_in = max(m["n_in"] for m in self.layer_meta)
        proj = new(T * n_in)
        mixw = max(L["mixer"]["heads"] * L["mixer"]["vdim"] for L in cfg.layers)
        mix = new(T * mixw)
        x = xs[0]
        ops.append(DeviceOp.embed(x, ctl, gl, GA.off["embed"], T, D, cfg.embedding_scale, wdt))
        layer_bufs = []
        shared: Dict[str, int] = {}

        def scratch(name, n):      # activations reused by every layer that needs them
            if name not in shared or sizes[shared[name]] < n:
                shared[name] = new(n)
            return shared[name]

        def next_x(cur):
            if keep_layers:
                return new(T * D)
            return xs[1] if cur == xs[0] else xs[0]

        # the norm that closes a sublayer (with the residual add) waits for the norm that opens the next one: one launch for both
        closing: List[tuple] = []

        def close_norm(nx, src, wb, w_off, res):
            flush()
            closing.append((nx, src, wb, w_off, res))

        def open_norm(dst, src, wb, w_off):
            if closing and closing[0][0] == src:
                nx, y_, cb, c_off, res = closing.pop()
                ops.append(DeviceOp.norm(nx, y_, cb, c_off, T, D, eps, wdt, res=res, then=dst, then_w=wb, then_w_off=w_off))
            else:
                flush()
                ops.append(DeviceOp.norm(dst, src, wb, w_off, T, D, eps, wdt))

        def flush():
            if closing:
                nx, y_, cb, c_off, res = closing.pop()
                ops.append(DeviceOp.norm(nx, y_, cb, c_off, T, D, eps, wdt, res=res))

        for i, L in enumerate(cfg.layers):
            m, meta, A, wb = L["mixer"], self.layer_meta[i], self.arenas[i], wbuf[i]
            H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            ni = meta["n_in"]
            open_norm(h, x, wb, A.off["norm1"])
            if L["type"] == "attention":
                ops.append(DeviceOp.linear(proj, h, wb, A.off["in"], T, ni, D, wdt, bias=wb, bias_off=A.off["in.b"]))
                win = m["mask"]["size"]
                ring = pool.buffers[f"l{i}.ring"]
                R = ring.elems // (pool.n_slots * G * dim)
                assert R >= win - 1 + T, "the session's key ring is shorter than window - 1 + chunk"
                table = new(win * H, self.bias_tables[i])
                ops.append(DeviceOp.window_attention(mix, proj, ext(ring), table, ctl, meta["q_off"], meta["k_off"], meta["g_off"],
                                                     T, H, G, dim, ni, win, R, m["scale"], m.get("softcap", 0.0)))
            else:
                ops.append(DeviceOp.linear(proj, h, wb, A.off["in"], T, ni, D, wdt))
                C, taps = meta["C"], meta["taps"]
                conv = scratch("conv", T * C)
                tail = ext(pool.buffers[f"l{i}.tail"]) if taps > 1 else ctl   # taps == 1: no carried inputs, the operand is unused
                ops.append(DeviceOp.causal_conv(conv, proj, wb, A.off["conv"], tail, ctl, T, C, taps, wdt, "silu", src_rs=ni))
                nag = H * dim + H * vdim
                ag = scratch("decay_gate", T * nag)     # [decay logits | gate logits] per token
                ops.append(DeviceOp.linear(ag, proj, wb, A.off["ag2"], T, nag, meta["ra"] + meta["rg"], wdt, src_off=meta["a1_off"], src_rs=ni))
                ops.append(DeviceOp.delta_rule(mix, conv, proj, ag, ag, wb, ext(pool.buffers[f"l{i}.S"]), ctl,
                                               0, G * dim, 2 * G * dim, meta["beta_off"], A.off["A_log"], A.off["dt_bias"], A.off["onorm"],
                                               T, H, G, dim, vdim, C, ni, nag, nag, wdt, eps, UNIT_EPS, dim ** -0.5, gate_off=H * dim))
            ops.append(DeviceOp.linear(y, mix, wb, A.off["o"], T, D, H * vdim, wdt))
            nx = next_x(x)
            close_norm(nx, y, wb, A.off["norm1b"], x)
            x = nx
            if L["mlp"] is not None:
                NE, E, ff, top = meta["NE"], meta["E"], meta["ff"], meta["top"]
                open_norm(h, x, wb, A.off["norm2"])
                rl, rt = scratch("router", T * NE), scratch("route", T * top * 2)
                ops.append(DeviceOp.linear(rl, h, wb, A.off["router"], T, NE, D, wdt))
                ops.append(DeviceOp.route(rt, rl, wb, A.off["correction"], T, NE, top, wdt))
                moe_op = DeviceOp.moe_ffn(y, h, rt, wb, 0, A.off["gate"], A.off["up"], A.off["down"], T, D, ff, E, top, wdt,
                                          meta["limit"], EXPERT_ALPHA)
                moe_op.u.seq.buf[4] = scratch("expert", seq_scratch_elems(moe_op))   # the library knows what its kernels stage
                ops.append(moe_op)
                nx = next_x(x)
                close_norm(nx, y, wb, A.off["norm2b"], x)
                x = nx
            layer_bufs.append(x)
        logits, rows = None, 0
        if head != "none":
            open_norm(h, x, gl, GA.off["final.norm"])
            rows = T if head == "all" else 1
            logits = new(rows * cfg.vocab)
            ops.append(DeviceOp.linear(logits, h, gl, GA.off["head"], rows, cfg.vocab, D, wdt, src_off=0 if head == "all" else (T - 1) * D))
        flush()
        prog = DeviceProgram(ops, sizes, uploads, [], externs)
        return LoweredProgram(prog, ctl, logits, rows, layer_bufs if keep_layers else None)

    def close(self):
        for b in self.buffers:
            b.free()
        self.buffers = []


def synthetic_config(width: int, n_layers: int, heads: int, kv_heads: int, dim: int, window: int, experts: int, top: int, ff: int,
                     vocab: int, identity: int = 1, attention_every: int = 2, conv: int = 4) -> dict:
    """config.json contents of a random-init model: every `attention_every`-th layer is a window-attention layer, the
    others are delta-rule layers; each has a routed feed-forward."""
    layers = []
    for i in range(n_layers):
        mlp = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "identity": identity, "top": top}}
        if i % attention_every == attention_every - 1:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window}, "bias_max": 4 * window,
                     "softcap": 30.0, "scale": dim ** -0.5}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        else:
            layers.append({"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv}, "mlp": mlp})
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "layers": layers}


def synthetic_tensors(cfg: dict, seed: int = 0, rank: int = 64, rel_rows: int = 32):
    """Accessor name -> random f32 tensor of the shape the configuration implies (benchmarks and smoke runs; values are
    scaled like a trained model's so that activations stay O(1))."""
    D = cfg["width"]

    def shape_of(name):
        if name in ("embed", "head"):
            return (cfg["vocab"], D)
        if name == "final.norm":
            return (D,)
        layer, rest = name.split(".", 1)
        L = cfg["layers"][int(layer[1:])]
        m = L["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if rest.startswith("norm"):
            return (D,)
        if rest.startswith("mlp."):
            r, ff = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            part = rest.split(".")[-1]
            return {"router": (r["experts"] + r["identity"], D), "correction": (r["experts"] + r["identity"],), "gate": (ff, D), "up": (ff, D),
                    "down": (D, ff)}[part]
        t = rest[len("mix."):]
        if L["type"] == "attention":
            return {"q": (H * d, D), "q.b": (H * d,), "k": (G * d, D), "k.b": (G * d,), "rel": (rel_rows, H), "g": (H * dv, D), "o": (D, H * dv)}[t]
        return {"q": (G * d, D), "k": (G * d, D), "v": (H * dv, D), "q.conv": (G * d, m["conv"]), "k.conv": (G * d, m["conv"]),
                "v.conv": (H * dv, m["conv"]), "b": (H, D), "A_log": (H,), "norm": (dv,), "a1": (rank, D), "a2": (H * d, rank),
                "dt_bias": (H * d,), "g1": (rank, D), "g2": (H * dv, rank), "o": (D, H * dv)}[t]

    def get(name):
        import zlib
        shp = shape_of(name)
        r = np.random.default_rng([seed, zlib.crc32(name.encode())])
        if name.endswith(("norm", "norm1", "norm2", "norm1b", "norm2b")):
            return np.ones(shp, np.float32)
        if len(shp) == 1:
            return (r.random(shp, dtype=np.float32) - 0.5) * 0.2
        a = r.random(shp, dtype=np.float32)
        a -= 0.5
        a *= np.float32(np.sqrt(12.0 / shp[1]))
        return a

    return get
