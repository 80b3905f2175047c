"""Plain, slow restatement of the Lududra decoder in numpy float64: one function per mechanism, written from
the design's equations and sharing no code with zgml_b200/.  Test infrastructure only.

Weights are a dict name -> float64 array with the checkpoint's tensor names; `cfg` is the parsed config.json.
Every function works token by token on purpose (the recurrences and the window are then impossible to get
wrong by a blocking argument); `forward` returns the logits and the residual stream after every layer.
"""
import math

import numpy as np


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def distance_bucket(n, n_rows, bias_max):
    """Row of the distance-bias table for distance n >= 0: exact for the first half of the rows, logarithmic
    up to bias_max for the second half."""
    half = n_rows // 2
    if n < half:
        return n
    return min(n_rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (n_rows - half))))


def window_attention(h, W, pre, m):
    """h [T, width] -> [T, width].  Keys double as values; a sink of score 0 sits in the softmax denominator."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    assert m["vdim"] == d
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(T, H, d)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(T, G, d)
    rel = W[pre + "rel"]
    gate = sigmoid(h @ W[pre + "g"].T).reshape(T, H, d)
    win, cap = m["mask"]["size"], m["softcap"]
    out = np.zeros((T, H, d))
    for i in range(T):
        lo = max(0, i - win + 1)
        for hh in range(H):
            kv = hh // (H // G)
            s = (k[lo:i + 1, kv] @ q[i, hh]) * m["scale"]
            s = cap * np.tanh(s / cap)
            s = s + np.array([rel[distance_bucket(i - j, rel.shape[0], m["bias_max"]), hh] for j in range(lo, i + 1)])
            mx = max(0.0, s.max())
            e = np.exp(s - mx)
            p = e / (math.exp(-mx) + e.sum())
            out[i, hh] = p @ k[lo:i + 1, kv]
    return (out * gate).reshape(T, H * d) @ W[pre + "o"].T


def causal_conv_silu(x, w):
    """x [T, C], w [C, taps] (last column = current token), zeros before the start; then SiLU."""
    T, C = x.shape
    taps = w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, C)), x], 0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += xp[j:j + T] * w[:, j]
    return y * sigmoid(y)


def channel_delta(h, W, pre, m, eps):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ W[pre + "q"].T, W[pre + "q.conv"]).reshape(T, G, d)
    k = causal_conv_silu(h @ W[pre + "k"].T, W[pre + "k.conv"]).reshape(T, G, d)
    v = causal_conv_silu(h @ W[pre + "v"].T, W[pre + "v.conv"]).reshape(T, H, dv)
    q = q / np.sqrt((q ** 2).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k ** 2).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[pre + "b"].T)                                             # [T, H]
    a = (h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "dt_bias"]               # [T, H * d]
    decay = np.exp(-np.exp(W[pre + "A_log"])[None, :, None] * softplus(a).reshape(T, H, d))
    gate = sigmoid((h @ W[pre + "g1"].T) @ W[pre + "g2"].T).reshape(T, H, dv)
    S = np.zeros((H, d, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hh in range(H):
            kv = hh // (H // G)
            S[hh] *= decay[t, hh][:, None]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, kv])
            S[hh] += np.outer(k[t, kv], u)
            o[t, hh] = S[hh].T @ q[t, kv]
    o = o / np.sqrt((o ** 2).mean(-1, keepdims=True) + eps) * W[pre + "norm"]
    return (o * gate).reshape(T, H * dv) @ W[pre + "o"].T


def route(h, W, pre, r):
    """-> (chosen expert indices [T, top], their weights [T, top]); indices >= experts are identity experts."""
    z = h @ W[pre + "router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    choice = s + W[pre + "correction"]
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :r["top"]]
    return idx, np.take_along_axis(s, idx, -1)


def expert(h, W, pre, limit):
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def moe(h, W, pre, mlp):
    r = mlp["router"]
    idx, wt = route(h, W, pre, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wt[t]):
            out[t] += w * (h[t] if e >= r["experts"] else expert(h[t], W, f"{pre}e{e}.", mlp["expert"]["limit"]))
    return out


def forward(cfg, W, tokens):
    """-> (logits [T, vocab], residual stream after every layer [layers, T, width])."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    stream = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, W[p + "norm1"], eps)
        if L["type"] == "attention":
            y = window_attention(h, W, p + "mix.", L["mixer"])
        elif L["type"] == "channel_delta":
            y = channel_delta(h, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + layer_norm(y, W[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            assert L["mlp"]["kind"] == "moe"
            y = moe(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp.", L["mlp"])
            x = x + layer_norm(y, W[p + "norm2b"], eps)
        stream.append(x.copy())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T, np.stack(stream)
