"""Small random Vemepel models for the tests: configurations of many shapes and bfloat16-exact random weights (so that the
device, whichever weight format it keeps, and the float64 restatement see the same numbers)."""
import numpy as np


def bf16_exact(x):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def diff_layer(heads=4, kv_heads=2, dim=8, vdim=12, block=7, diff=0.4, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": block}, "diff": diff,
         "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent_layer(heads=3, dim=10, vdim=6, kv_rank=14, scale=None, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale if scale is not None else dim ** -0.5}}


def latent2_layer(heads=3, dim=10, rot_dim=6, vdim=8, kv_rank=12, base=500.0, scale=None, mlp=None):
    return {"type": "latent_attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim},
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, width=40, vocab=61, eps=1e-5, logit_scale=1.5):
    return {"architecture": "Vemepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def random_weights(cfg, seed=0, qk_gain=1.0):
    """name -> float32 array (bfloat16-exact).  `qk_gain` scales the query side of every mixer: large values make the softmax
    peaky, so a key wrongly inside or outside a mask, or a lost cache row, moves the output a lot."""
    r = np.random.default_rng(seed)
    D, W = cfg["width"], {}

    def lin(n_out, n_in, gain=1.0):
        return r.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)

    def around_zero(n):
        return 0.2 * r.standard_normal(n)

    W["embed"] = r.standard_normal((cfg["vocab"], D))
    W["head"] = lin(cfg["vocab"], D)
    W["final.norm"] = around_zero(D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        W[p + "norm1"], W[p + "norm1b"] = around_zero(D), around_zero(D)
        W[p + "shift"] = r.uniform(0.0, 1.0, D)
        W[p + "dwa"] = np.concatenate([0.3 * r.standard_normal(i + 1), [1.0 + 0.1 * r.standard_normal()]])
        if L["type"] == "attention":
            G = m["kv_heads"]
            W[p + "mix.q"] = lin(H * 2 * d, D, qk_gain)
            if m.get("kv_from") is None:
                W[p + "mix.k"], W[p + "mix.v"] = lin(G * 2 * d, D, 1.5), lin(G * dv, D)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[p + "mix." + n] = 0.3 * r.standard_normal(d)
        else:
            rd = m.get("rot_dim", 0)
            rank = m["kv_rank"]
            W[p + "mix.q"] = lin(H * (d + rd), D, qk_gain)
            W[p + "mix.dkv"] = lin(rank + rd, D, 1.5)
            W[p + "mix.dkv.norm"] = 1.0 + 0.2 * r.standard_normal(rank)
            W[p + "mix.uk"], W[p + "mix.uv"] = lin(H * d, rank), lin(H * dv, rank)
            W[p + "mix.g"] = lin(H * dv if L["type"] == "latent_attention_2" else H, D, 2.0)
        W[p + "mix.o"] = lin(D, H * dv)
        mlp = L["mlp"]
        if mlp is not None:
            W[p + "norm2"], W[p + "norm2b"] = around_zero(D), around_zero(D)
            if mlp["kind"] == "dense":
                W[p + "mlp.up"], W[p + "mlp.down"] = lin(mlp["ff"], D, 1.5), lin(D, mlp["ff"])
                W[p + "mlp.act"] = np.array([0.7, -0.4, 0.3, 0.1]) + 0.1 * r.standard_normal(4)
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                W[p + "mlp.router"] = lin(E, D, 3.0)
                W[p + "mlp.router.b"] = 0.5 * r.standard_normal(E)
                for e in range(E):
                    W[p + f"mlp.e{e}.gate"], W[p + f"mlp.e{e}.up"] = lin(ff, D, 2.0), lin(ff, D, 2.0)
                    W[p + f"mlp.e{e}.down"] = lin(D, ff)
    return {k: bf16_exact(np.asarray(v, dtype=np.float32)) for k, v in W.items()}


def as_f64(W):
    return {k: v.astype(np.float64) for k, v in W.items()}
