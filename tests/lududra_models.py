"""Small random Lududra models for the tests: configurations of many shapes and bfloat16-exact random weights
(so that the device, whichever weight format it keeps, and the float64 restatement see the same numbers)."""
import numpy as np


def bf16_exact(x):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def attention_layer(heads=4, kv_heads=2, dim=16, window=8, rel_rows=8, bias_max=32, softcap=30.0, scale=None, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window}, "bias_max": bias_max,
                      "softcap": softcap, "scale": scale if scale is not None else dim ** -0.5, "_rel_rows": rel_rows}}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, rank_a=4, rank_g=6, mlp=None):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "_rank_a": rank_a, "_rank_g": rank_g}}


def moe(experts=6, identity=1, top=2, ff=24, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


def config(layers, width=48, vocab=97, eps=1e-5, embed_scale=0.7):
    return {"architecture": "Lududra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "layers": layers}


def random_weights(cfg, seed=0, qk_gain=1.0):
    """name -> float32 array (bfloat16-exact).  `qk_gain` scales the attention's query and key projections: large values
    make the softmax peaky, so a key wrongly inside or outside the window, or a missing sink, moves the output a lot."""
    r = np.random.default_rng(seed)
    D, W = cfg["width"], {}

    def lin(n_out, n_in, gain=1.0):
        return r.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)

    def gamma(n):
        return 1.0 + 0.2 * r.standard_normal(n)

    W["embed"] = r.standard_normal((cfg["vocab"], D))
    W["head"] = lin(cfg["vocab"], D)
    W["final.norm"] = gamma(D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[p + "norm1"], W[p + "norm1b"] = gamma(D), gamma(D)
        if L["type"] == "attention":
            W[p + "mix.q"], W[p + "mix.k"] = lin(H * d, D, qk_gain), lin(G * d, D, qk_gain)
            W[p + "mix.q.b"], W[p + "mix.k.b"] = 0.3 * r.standard_normal(H * d), 0.3 * r.standard_normal(G * d)
            W[p + "mix.rel"] = r.standard_normal((m["_rel_rows"], H))
            W[p + "mix.g"] = lin(H * dv, D)
        else:
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = lin(G * d, D), lin(G * d, D), lin(H * dv, D)
            for n, c in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[p + f"mix.{n}.conv"] = 0.6 * r.standard_normal((c, m["conv"]))
            W[p + "mix.b"] = lin(H, D)
            W[p + "mix.A_log"] = r.uniform(-1.5, 0.5, H)
            W[p + "mix.dt_bias"] = r.uniform(-2.0, 1.0, H * d)
            W[p + "mix.norm"] = gamma(dv)
            W[p + "mix.a1"], W[p + "mix.a2"] = lin(m["_rank_a"], D), lin(H * d, m["_rank_a"], 2.0)
            W[p + "mix.g1"], W[p + "mix.g2"] = lin(m["_rank_g"], D), lin(H * dv, m["_rank_g"], 2.0)
        W[p + "mix.o"] = lin(D, H * dv)
        if L["mlp"] is not None:
            rt, ff = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            W[p + "norm2"], W[p + "norm2b"] = gamma(D), gamma(D)
            W[p + "mlp.router"] = lin(rt["experts"] + rt["identity"], D, 3.0)
            W[p + "mlp.correction"] = 0.05 * r.standard_normal(rt["experts"] + rt["identity"])
            for e in range(rt["experts"]):
                W[p + f"mlp.e{e}.gate"], W[p + f"mlp.e{e}.up"] = lin(ff, D, 2.0), lin(ff, D, 2.0)
                W[p + f"mlp.e{e}.down"] = lin(D, ff)
    return {k: bf16_exact(v.astype(np.float32)) for k, v in W.items()}


def as_f64(W):
    return {k: v.astype(np.float64) for k, v in W.items()}
