"""Vemepel: a decoder-only stack whose layers pair a token mixer — differential attention inside position blocks (with
grouped key / value heads, optionally borrowing another layer's keys and values), or latent attention (keys and values
expanded per head from one cached latent, with or without a rotated key part shared by all heads) — with a PolyNorm
feed-forward or a routed mixture of gated experts.  Every sublayer sits between an RMS norm before and one after it; the
mixer's input is token-shifted; each layer's input is a learned average over the outputs of all earlier layers.

This file is the model's configuration reader, its weight packer and its LOWERING to a DeviceProgram; the arithmetic is in
the sequence-model DeviceOps of the CUDA library (csrc/seqops.cu, csrc/mixops.cu) and all state in the session's
`SequenceStatePool`.  Every size and per-model constant comes from config.json or a tensor's shape.

Per layer (x: f32 stream entering the layer, X_j: result of layer j - 1, X_0 the embedding):
    h = shift(RMS(x; 1 + norm1));  x = x + RMS(mixer(h); 1 + norm1b);  x = x + RMS(ff(RMS(x; 1 + norm2)); 1 + norm2b);  X_{i+1} = x
    next x = sum_j dwa[j] X_j

attention          [q | k | v] = W h in ONE matmul; k | v join the layer's cache; CACHED_ATTENTION with two score maps per
                   head and a block mask; MAP_COMBINE (a1 - lambda a2, unit RMS per head, times 1 - diff); W_o.  lambda is
                   a constant of the checkpoint and is evaluated in f32 at load.  A borrowing layer projects q only and
                   attends over the owner's cache.
latent attention   [q | dkv | gate] = W h in ONE matmul; CACHE_APPEND norms the latent (and rotates the shared key part)
                   on its way into the cache.  Attention runs in the ABSORBED form: per head q' = W_uk^T q (HEAD_LINEAR
                   over the transposed up-projection), scores and the weighted sum are taken against the cached latent
                   itself (one key / value head of kv_rank (+ rot_dim) columns serving all heads), and the value
                   up-projection is applied to the result (HEAD_LINEAR, the sigmoid gate in its epilogue), so nothing per head
                   is ever cached or re-expanded.
feed-forward       dense: W_up, POLY_NORM, W_down.  moe: router matmul, ROUTE (bias added, top-k, softmax over the chosen),
                   MOE_FFN over stacked expert weights.
"""
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import abi
from ..backend import CudaBackend, DeviceBuffer, DeviceOp, DeviceProgram, ExternBuffer, ProgramIO, seq_scratch_elems
from .safetensors import SafetensorsFile
from .session import LoweredProgram
from .state import SequenceStatePool, StateSpec
from .weights import WeightArena

ARCHITECTURE = "Vemepel"
DEFAULT_CONTEXT = 4096     # positions a sequence may reach when the caller names no bound
MIXERS = ("attention", "latent_attention", "latent_attention_2")


@dataclass(frozen=True)
class VemepelConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: tuple            # of dicts: {"type", "mixer": {...}, "mlp": {...} | None}

    @classmethod
    def from_dict(cls, c: dict) -> "VemepelConfig":
        if c.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture = {c.get('architecture')!r}")
        layers = []
        for i, L in enumerate(c["layers"]):
            m = dict(L["mixer"])
            kind = L["type"]
            if kind not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            if kind == "attention":
                if m["heads"] % m["kv_heads"]:
                    raise ValueError(f"layer {i}: heads not a multiple of kv_heads")
                if m["mask"]["size"] < 1:
                    raise ValueError(f"layer {i}: block size must be positive")
                src = m.get("kv_from")
                if src is not None:
                    if not (0 <= src < i) or c["layers"][src]["type"] != "attention" or c["layers"][src]["mixer"].get("kv_from") is not None:
                        raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with projections of its own")
                    o = c["layers"][src]["mixer"]
                    if (o["kv_heads"], o["dim"], o["vdim"]) != (m["kv_heads"], m["dim"], m["vdim"]):
                        raise ValueError(f"layer {i}: key / value shape differs from layer {src}'s")
            elif kind == "latent_attention_2":
                if m["rot"]["dims"] != m["rot_dim"] or m["rot_dim"] % 2:
                    raise ValueError(f"layer {i}: the rotated part must be rot_dim = rot.dims (even) wide")
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            if mlp is not None and mlp["kind"] == "moe" and not (1 <= mlp["router"]["top"] <= mlp["router"]["experts"]):
                raise ValueError(f"layer {i}: top must lie in 1 .. experts")
            layers.append({"type": kind, "mixer": m, "mlp": mlp})
        return cls(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), float(c.get("logit_scale", 1.0)), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "VemepelConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


def differential_lambda(lq1, lk1, lq2, lk2, diff: float) -> float:
    """exp(lq1 . lk1) - exp(lq2 . lk2) + diff, in f32 like every other scalar of the attention."""
    f = np.float32
    d1 = np.sum(lq1.astype(f) * lk1.astype(f), dtype=f)
    d2 = np.sum(lq2.astype(f) * lk2.astype(f), dtype=f)
    return float(f(np.exp(d1)) - f(np.exp(d2)) + f(diff))


class VemepelModel:
    """Weights resident in HBM (one arena per layer + one for embedding / final norm / head) and the lowering."""

    bounded_context = True     # latent layers cache every position: a sequence cannot outgrow the cache

    def __init__(self, be: CudaBackend, cfg: VemepelConfig, tensors, dtype: str = "bfloat16"):
        """tensors: name -> f32 array accessor (`tensors(name)`), e.g. SafetensorsFile.f32."""
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.be, self.cfg, self.dtype = be, cfg, dtype
        self.wdt = abi.W_BF16 if dtype == "bfloat16" else abi.W_F32
        self.vocab, self.width = cfg.vocab, cfg.width
        self.layer_meta: List[dict] = []
        self.arenas: List[WeightArena] = []
        self.buffers: List[DeviceBuffer] = []
        D = cfg.width
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L["mixer"]
            A = WeightArena(self.wdt)
            meta = {"type": L["type"]}
            for n in ("norm1", "norm1b", "shift"):
                t = tensors(p + n)
                assert t.shape == (D,), f"{p + n}: shape {t.shape}"
                A.add(n, t)
            dwa = tensors(p + "dwa")
            assert dwa.shape == (i + 2,), f"{p}dwa: shape {dwa.shape}"
            if i:      # the average that ENTERS this layer is taken by its opening norm: the previous layer's coefficients live here
                A.add("avg_in", tensors(f"l{i - 1}.dwa"))
            H, dim, vdim = m["heads"], m["dim"], m["vdim"]
            if L["type"] == "attention":
                G = m["kv_heads"]
                q = tensors(p + "mix.q")
                assert q.shape == (H * 2 * dim, D)
                owner = m.get("kv_from")
                if owner is None:
                    k, v = tensors(p + "mix.k"), tensors(p + "mix.v")
                    assert k.shape == (G * 2 * dim, D) and v.shape == (G * vdim, D)
                    A.add("in", np.concatenate([q, k, v], 0))
                    meta.update(n_in=(H + G) * 2 * dim + G * vdim, owner=i)
                else:
                    A.add("in", q)
                    meta.update(n_in=H * 2 * dim, owner=owner)
                meta["lambda"] = differential_lambda(*(tensors(p + f"mix.{n}") for n in ("lq1", "lk1", "lq2", "lk2")), m["diff"])
            else:
                rank = m["kv_rank"]
                rd = m["rot_dim"] if L["type"] == "latent_attention_2" else 0
                ng = H * vdim if L["type"] == "latent_attention_2" else H       # gate per element / per head
                q, dkv, g = tensors(p + "mix.q"), tensors(p + "mix.dkv"), tensors(p + "mix.g")
                uk, uv = tensors(p + "mix.uk"), tensors(p + "mix.uv")
                assert q.shape == (H * (dim + rd), D) and dkv.shape == (rank + rd, D) and g.shape == (ng, D)
                assert uk.shape == (H * dim, rank) and uv.shape == (H * vdim, rank)
                A.add("in", np.concatenate([q, dkv, g], 0))
                A.add("dkv.norm", tensors(p + "mix.dkv.norm"))
                A.add("ukT", uk.reshape(H, dim, rank).transpose(0, 2, 1))      # [H, rank, dim]: q' = W_uk^T q per head
                A.add("uv", uv)                                                  # [H, vdim, rank]
                meta.update(n_in=H * (dim + rd) + rank + rd + ng, rank=rank, rd=rd, ng=ng, dkv_off=H * (dim + rd), g_off=H * (dim + rd) + rank + rd)
            o = tensors(p + "mix.o")
            assert o.shape == (D, H * vdim)
            A.add("o", o)
            mlp = L["mlp"]
            if mlp is not None:
                A.add("norm2", tensors(p + "norm2"))
                A.add("norm2b", tensors(p + "norm2b"))
                if mlp["kind"] == "dense":
                    up, down, act = tensors(p + "mlp.up"), tensors(p + "mlp.down"), tensors(p + "mlp.act")
                    ff = up.shape[0]
                    assert up.shape == (ff, D) and down.shape == (D, ff) and act.shape == (4,) and ff == mlp.get("ff", ff)
                    A.add("up", up)
                    A.add("down", down)
                    A.add("act", act)
                    meta.update(ff=ff)
                else:
                    E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
                    router = tensors(p + "mlp.router")
                    assert router.shape == (E, D)
                    A.add("router", router)
                    A.add("router.b", tensors(p + "mlp.router.b"))
                    for part, shape in (("gate", (ff, D)), ("up", (ff, D)), ("down", (D, ff))):
                        stack = [tensors(p + f"mlp.e{e}.{part}") for e in range(E)]
                        assert all(s.shape == shape for s in stack)
                        A.add(part, np.stack(stack))
                    meta.update(E=E, top=top, ff=ff)
            self.layer_meta.append(meta)
            self.arenas.append(A)
            self.buffers.append(A.upload(be))
        A = WeightArena(self.wdt)
        emb, head = tensors("embed"), tensors("head")
        assert emb.shape == (cfg.vocab, D) and head.shape == (cfg.vocab, D)
        A.add("embed", emb)
        A.add("final.norm", tensors("final.norm"))
        A.add("avg_in", tensors(f"l{len(cfg.layers) - 1}.dwa"))
        A.add("head", head)
        self.arenas.append(A)
        self.buffers.append(A.upload(be))

    @classmethod
    def load(cls, be: CudaBackend, model_dir: str, dtype: str = "bfloat16") -> "VemepelModel":
        cfg = VemepelConfig.from_json(os.path.join(model_dir, "config.json"))
        sf = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
        try:
            return cls(be, cfg, sf.f32, dtype)
        finally:
            sf.close()

    def weight_bytes(self) -> int:
        return sum(b.nbytes for b in self.buffers)

    # ── state ──
    def _cache_rows(self, i: int, max_chunk: int, capacity: int) -> int:
        """Rows of the cache layer i owns: what the masks of its readers (itself and the layers that borrow from it) can reach
        back plus one step — position p lives in row p mod rows — and never more than one row per position."""
        if self.cfg.layers[i]["type"] != "attention":
            return capacity
        reach = max(L["mixer"]["mask"]["size"] - 1 + max_chunk for L, M in zip(self.cfg.layers, self.layer_meta) if M["type"] == "attention" and M["owner"] == i)
        return min(reach, capacity)

    def state_specs(self, max_chunk: int, max_context: Optional[int] = None) -> List[StateSpec]:
        capacity = self.capacity(max_chunk, max_context)
        specs = []
        for i, L in enumerate(self.cfg.layers):
            m, M = L["mixer"], self.layer_meta[i]
            specs.append(StateSpec(f"l{i}.shift", self.width, True))
            if L["type"] == "attention":
                if M["owner"] == i:
                    specs.append(StateSpec(f"l{i}.kv", self._cache_rows(i, max_chunk, capacity) * m["kv_heads"] * (2 * m["dim"] + m["vdim"]), False))
            else:
                specs.append(StateSpec(f"l{i}.latent", capacity * (M["rank"] + M["rd"]), False))
        return specs

    @staticmethod
    def capacity(max_chunk: int, max_context: Optional[int]) -> int:
        return max(int(max_context) if max_context else DEFAULT_CONTEXT, max_chunk)

    # ── lowering ──
    def lower(self, T: int, head: str, pool: SequenceStatePool, keep_layers: bool = False) -> LoweredProgram:
        cfg, wdt, D, eps = self.cfg, self.wdt, self.cfg.width, self.cfg.norm_eps
        nL = len(cfg.layers)
        sizes: List[int] = []
        uploads: List[ProgramIO] = []
        externs: List[ExternBuffer] = []
        ops = []

        def new(n):
            sizes.append(max(int(n), 1))
            return len(sizes) - 1

        ext_of: Dict[int, int] = {}

        def ext(buf: DeviceBuffer):      # one program buffer per device buffer, so that layers sharing a cache are ordered
            if id(buf) not in ext_of:
                sizes.append(buf.elems)
                externs.append(ExternBuffer(len(sizes) - 1, buf))
                ext_of[id(buf)] = len(sizes) - 1
            return ext_of[id(buf)]

        ctl = new(abi.CTL_IDS + T)
        wbuf = [ext(b) for b in self.buffers]
        gl, GA = wbuf[-1], self.arenas[-1]
        TD = T * D
        hist = new((nL + 1) * TD)                  # X_0 .. X_nL, the terms of the depth average
        xa = new(TD)                               # the stream after the mixer's sublayer
        h0, h, y = new(TD), new(TD), new(TD)
        proj = new(T * max(m["n_in"] for m in self.layer_meta))
        mix = new(T * max(L["mixer"]["heads"] * L["mixer"]["vdim"] for L in cfg.layers))
        shared: Dict[str, int] = {}

        def scratch(name, n):      # activations reused by every layer that needs them
            if name not in shared or sizes[shared[name]] < n:
                shared[name] = new(n)
            return shared[name]

        ops.append(DeviceOp.embed(hist, ctl, gl, GA.off["embed"], T, D, 1.0, wdt))
        x = hist                                   # layer 0 reads X_0 in place (offset 0 of the history)
        xm = new(TD)                               # the depth average that enters every later layer
        layer_bufs = []
        slots = pool.n_slots
        for i, L in enumerate(cfg.layers):
            m, meta, A, wb = L["mixer"], self.layer_meta[i], self.arenas[i], wbuf[i]
            H, dim, vdim = m["heads"], m["dim"], m["vdim"]
            ni = meta["n_in"]
            shift_state = ext(pool.buffers[f"l{i}.shift"])
            # The opening norm also takes the depth average that enters the layer (layer 0 reads the embedding itself) and, in
            # single-token steps, shifts its own row against the carried one: one launch.
            average = None
            if i:
                x = new(TD) if keep_layers else xm
                average = (x, A.off["avg_in"], i + 1, TD)
                layer_bufs.append(x)
            src = hist
            if T == 1:
                ops.append(DeviceOp.norm(h, src, wb, A.off["norm1"], T, D, eps, wdt, kind="rms1", shift_state=shift_state, shift_off=A.off["shift"], ctl=ctl, average=average))
            else:
                ops.append(DeviceOp.norm(h0, src, wb, A.off["norm1"], T, D, eps, wdt, kind="rms1", average=average))
                ops.append(DeviceOp.token_shift(h, h0, wb, A.off["shift"], shift_state, ctl, T, D, wdt))
            ops.append(DeviceOp.linear(proj, h, wb, A.off["in"], T, ni, D, wdt))
            if L["type"] == "attention":
                G = m["kv_heads"]
                cache = pool.buffers[f"l{meta['owner']}.kv"]
                width = G * (2 * dim + vdim)
                R = cache.elems // (slots * width)
                if meta["owner"] == i:
                    ops.append(DeviceOp.cache_append(ext(cache), proj, ctl, H * 2 * dim, 0, T, width, ni, width, R))
                att = scratch("maps", T * H * 2 * vdim)
                ops.append(DeviceOp.cached_attention(att, proj, ext(cache), ext(cache), ctl, 0, 0, G * 2 * dim, T, H, G, 2, dim, vdim, ni, width, width,
                                                     R, m["scale"], mask="block", mask_size=m["mask"]["size"]))
                ops.append(DeviceOp.map_combine(mix, att, T * H, vdim, meta["lambda"], eps, 1.0 - m["diff"]))
            else:
                rank, rd = meta["rank"], meta["rd"]
                cw = rank + rd
                cache = pool.buffers[f"l{i}.latent"]
                R = cache.elems // (slots * cw)
                ops.append(DeviceOp.cache_append(ext(cache), proj, ctl, meta["dkv_off"], 0, T, cw, ni, cw, R, norm_w=wb, norm_off=A.off["dkv.norm"],
                                                 normed=rank, eps=eps, wdt=wdt, rot=rd, rot_base=m["rot"]["base"] if rd else 0.0))
                qa = scratch("absorbed_q", T * H * cw)
                ops.append(DeviceOp.head_linear(qa, proj, wb, A.off["ukT"], T, H, rank, dim, wdt, src_col=0, src_hs=dim + rd, src_rs=ni, dst_hs=cw, dst_rs=H * cw))
                if rd:
                    ops.append(DeviceOp.rotary(qa, ctl, rank, T, H, cw, H * cw, rd, m["rot"]["base"], src=proj, src_col=dim, src_hs=dim + rd, src_rs=ni))
                lat = scratch("latent_out", T * H * rank)
                ops.append(DeviceOp.cached_attention(lat, qa, ext(cache), ext(cache), ctl, 0, 0, 0, T, H, 1, 1, cw, rank, H * cw, cw, cw, R, m["scale"]))
                # the value up-projection, with the output gate (one per head, or one per element) in its epilogue
                ops.append(DeviceOp.head_linear(mix, lat, wb, A.off["uv"], T, H, vdim, rank, wdt, gate=proj, gate_col=meta["g_off"], gate_rs=ni,
                                                gate_group=vdim if meta["ng"] == H else 1))
            ops.append(DeviceOp.linear(y, mix, wb, A.off["o"], T, D, H * vdim, wdt))
            mlp = L["mlp"]
            out_off = (i + 1) * TD
            if mlp is None:
                ops.append(DeviceOp.norm(hist, y, wb, A.off["norm1b"], T, D, eps, wdt, kind="rms1", res=x, dst_off=out_off))
            else:
                # the norm that closes the mixer's sublayer (with the residual add) and the one that opens the feed-forward: one launch
                ops.append(DeviceOp.norm(xa, y, wb, A.off["norm1b"], T, D, eps, wdt, kind="rms1", res=x, then=h, then_w=wb, then_w_off=A.off["norm2"],
                                         then_kind="rms1"))
                if mlp["kind"] == "dense":
                    ff = meta["ff"]
                    u = scratch("ff", T * ff)
                    ops.append(DeviceOp.linear(u, h, wb, A.off["up"], T, ff, D, wdt))
                    ops.append(DeviceOp.poly_norm(u, u, wb, A.off["act"], T, ff, eps, wdt))
                    ops.append(DeviceOp.linear(y, u, wb, A.off["down"], T, D, ff, wdt))
                else:
                    E, ff, top = meta["E"], meta["ff"], meta["top"]
                    rl, rt = scratch("router", T * E), scratch("route", T * top * 2)
                    ops.append(DeviceOp.linear(rl, h, wb, A.off["router"], T, E, D, wdt))
                    ops.append(DeviceOp.route(rt, rl, wb, A.off["router.b"], T, E, top, wdt, mode="biased_top"))
                    moe_op = DeviceOp.moe_ffn(y, h, rt, wb, 0, A.off["gate"], A.off["up"], A.off["down"], T, D, ff, E, top, wdt, float("inf"), 1.0,
                                              up_offset=0.0)
                    moe_op.u.seq.buf[4] = scratch("expert", seq_scratch_elems(moe_op))   # the library knows what its kernels stage
                    ops.append(moe_op)
                ops.append(DeviceOp.norm(hist, y, wb, A.off["norm2b"], T, D, eps, wdt, kind="rms1", res=xa, dst_off=out_off))
        logits, rows = None, 0
        x = new(TD) if keep_layers else xm          # the average over all layers: what the head reads
        layer_bufs.append(x)
        if head != "none":
            ops.append(DeviceOp.norm(h, hist, gl, GA.off["final.norm"], T, D, eps, wdt, kind="rms1", gain=cfg.logit_scale, average=(x, GA.off["avg_in"], nL + 1, TD)))
            rows = T if head == "all" else 1
            logits = new(rows * cfg.vocab)
            ops.append(DeviceOp.linear(logits, h, gl, GA.off["head"], rows, cfg.vocab, D, wdt, src_off=0 if head == "all" else (T - 1) * D))
        elif keep_layers:
            ops.append(DeviceOp.depth_mix(x, hist, gl, GA.off["avg_in"], TD, nL + 1, TD, wdt))
        prog = DeviceProgram(ops, sizes, uploads, [], externs)
        return LoweredProgram(prog, ctl, logits, rows, layer_bufs if keep_layers else None)

    def close(self):
        for b in self.buffers:
            b.free()
        self.buffers = []


def synthetic_config(width: int, n_layers: int, heads: int, kv_heads: int, dim: int, block: int, experts: int, top: int, ff: int, vocab: int,
                     kv_rank: int = 512, rot_dim: int = 64) -> dict:
    """config.json contents of a random-init model: the layers cycle through differential attention (grouped heads, two maps of
    dim / 2 each, every second one borrowing the keys and values of the one before), latent attention with a rotated key
    part and latent attention without; feed-forwards alternate between routed experts and a dense PolyNorm layer as wide as
    the experts a token uses."""
    layers, last_owner = [], None
    for i in range(n_layers):
        mlp = ({"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}} if i % 2 == 0 else {"kind": "dense", "ff": top * ff})
        kind = i % 3
        if kind == 0:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim // 2, "vdim": dim, "mask": {"size": block}, "diff": 0.5, "scale": (dim // 2) ** -0.5}
            if last_owner is not None:
                mixer["kv_from"], last_owner = last_owner, None
            else:
                last_owner = i
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        elif kind == 1:
            mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": dim, "kv_rank": kv_rank, "rot": {"base": 10000.0, "dims": rot_dim},
                     "scale": (dim + rot_dim) ** -0.5}
            layers.append({"type": "latent_attention_2", "mixer": mixer, "mlp": mlp})
        else:
            layers.append({"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": kv_rank, "scale": dim ** -0.5}, "mlp": mlp})
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 1.0, "layers": layers}


def synthetic_tensors(cfg: dict, seed: int = 0):
    """Accessor name -> random f32 tensor of the shape the configuration implies (benchmarks and smoke runs; values are
    scaled like a trained model's so that activations stay O(1))."""
    D = cfg["width"]

    def shape_of(name):
        if name in ("embed", "head"):
            return (cfg["vocab"], D)
        if name == "final.norm":
            return (D,)
        layer, rest = name.split(".", 1)
        i = int(layer[1:])
        L = cfg["layers"][i]
        m = L["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if rest.startswith("norm") or rest == "shift":
            return (D,)
        if rest == "dwa":
            return (i + 2,)
        if rest.startswith("mlp."):
            part = rest.split(".", 1)[1]
            if L["mlp"]["kind"] == "dense":
                return {"up": (L["mlp"]["ff"], D), "down": (D, L["mlp"]["ff"]), "act": (4,)}[part]
            E, ff = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            return {"router": (E, D), "router.b": (E,), "gate": (ff, D), "up": (ff, D), "down": (D, ff)}[part.split(".")[-1] if part.startswith("e") else part]
        t = rest[len("mix."):]
        if L["type"] == "attention":
            G = m["kv_heads"]
            return {"q": (H * 2 * d, D), "k": (G * 2 * d, D), "v": (G * dv, D), "lq1": (d,), "lk1": (d,), "lq2": (d,), "lk2": (d,), "o": (D, H * dv)}[t]
        rd, rank = m.get("rot_dim", 0), m["kv_rank"]
        return {"q": (H * (d + rd), D), "dkv": (rank + rd, D), "dkv.norm": (rank,), "uk": (H * d, rank), "uv": (H * dv, rank),
                "g": (H * dv if L["type"] == "latent_attention_2" else H, D), "o": (D, H * dv)}[t]

    def get(name):
        import zlib
        shp = shape_of(name)
        r = np.random.default_rng([seed, zlib.crc32(name.encode())])
        if name.endswith("dkv.norm"):
            return np.ones(shp, np.float32)
        if name.endswith(".dwa"):
            a = np.full(shp, 0.1 / shp[0], np.float32)
            a[-1] = 1.0
            return a
        if name.endswith(".act"):
            return np.array([0.6, 0.3, 0.1, 0.0], np.float32)
        if name.endswith(".shift"):
            return r.random(shp, dtype=np.float32)
        if len(shp) == 1:
            return (r.random(shp, dtype=np.float32) - 0.5) * 0.2
        a = r.random(shp, dtype=np.float32)
        a -= 0.5
        a *= np.float32(np.sqrt(12.0 / shp[1]))
        return a

    return get
