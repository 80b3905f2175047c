"""Float64 restatement of the Vemepel design from its equations: one function per mechanism, whole sequences at once,
plain NumPy.  It shares no code with zgml_b200/; the GPU tests compare the framework against it.

Notation: x [T, D] residual stream, h the mixer's (or feed-forward's) input, W[name] the checkpoint tensors ([out, in]
matrices applied as W h), p the position of a token in its sequence (from 0).
"""
import numpy as np


def rms_norm(x, eps, weight=None, unit_offset=False):
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` (or 1 + weight when it is stored around zero)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    if weight is None:
        return y
    return y * ((1.0 + weight) if unit_offset else weight)


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu with h_{-1} = 0; the previous token's h is the one before this replacement."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def depth_average(history, coeff):
    """sum_j coeff[j] * history[j] over the embedding output and every layer result so far."""
    assert len(history) == len(coeff)
    return sum(c * X for c, X in zip(coeff, history))


def rotate_interleaved(x, positions, dims, base):
    """Rotary positions on the first `dims` entries of the last axis of x [T, ..., n]: (x[2i], x[2i+1]) turns by the angle
    p * base^(-2i / dims)."""
    out = x.copy()
    i = np.arange(dims // 2)
    freq = base ** (-2.0 * i / dims)
    ang = positions[:, None].astype(np.float64) * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def causal_mask(T):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return j <= i


def chunk_mask(T, size):
    """Causal inside blocks of `size` positions counted from position 0."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_attention(q, k, v, visible, scale):
    """q [T, dk], k [T, dk], v [T, dv], visible [T, T] bool -> [T, dv]; ordinary softmax over the visible keys."""
    s = (q @ k.T) * scale
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    w = w / w.sum(axis=-1, keepdims=True)
    return w @ v


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def latent_attention(h, W, p, m, eps):
    """Keys and values expanded per head from one normed latent; no positions; one sigmoid gate per head."""
    T = h.shape[0]
    H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[p + "q"].T).reshape(T, H, dim)
    c = rms_norm(h @ W[p + "dkv"].T, eps, W[p + "dkv.norm"])
    assert c.shape[1] == rank
    k = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vdim)
    gate = sigmoid(h @ W[p + "g"].T)                       # [T, H]
    vis = causal_mask(T)
    out = np.stack([softmax_attention(q[:, a], k[:, a], v[:, a], vis, m["scale"]) * gate[:, a:a + 1] for a in range(H)], 1)
    return out.reshape(T, H * vdim) @ W[p + "o"].T


def latent_attention_2(h, W, p, m, eps):
    """Latent attention with a rotated key part shared by all heads; elementwise sigmoid gate on the concatenated heads."""
    T = h.shape[0]
    H, dim, rd, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    assert m["rot"]["dims"] == rd
    pos = np.arange(T)
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate_interleaved(q[..., dim:], pos, rd, m["rot"]["base"])
    d = h @ W[p + "dkv"].T
    assert d.shape[1] == rank + rd
    c = rms_norm(d[:, :rank], eps, W[p + "dkv.norm"])
    k_rot = rotate_interleaved(d[:, rank:], pos, rd, m["rot"]["base"])
    k = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vdim)
    vis = causal_mask(T)
    heads = []
    for a in range(H):
        qa = np.concatenate([q_plain[:, a], q_rot[:, a]], 1)
        ka = np.concatenate([k[:, a], k_rot], 1)
        heads.append(softmax_attention(qa, ka, v[:, a], vis, m["scale"]))
    out = np.stack(heads, 1).reshape(T, H * vdim) * sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def differential_lambda(W, p, diff):
    return np.exp(np.sum(W[p + "lq1"] * W[p + "lk1"])) - np.exp(np.sum(W[p + "lq2"] * W[p + "lk2"])) + diff


def keys_values(h, W, p, m):
    """The projections of a differential-attention layer that owns its keys and values: k [T, G, 2, dim], v [T, G, vdim]."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    return (h @ W[p + "k"].T).reshape(T, G, 2, dim), (h @ W[p + "v"].T).reshape(T, G, vdim)


def differential_attention(h, W, p, m, eps, kv):
    """Two softmax maps per head over the same values, o = a1 - lambda a2, unit RMS per head, times (1 - diff); grouped
    key / value heads; causal inside position blocks.  `kv` = (k, v) of this layer or of the layer it borrows from."""
    T = h.shape[0]
    H, G, dim, vdim, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    q = (h @ W[p + "q"].T).reshape(T, H, 2, dim)
    k, v = kv
    lam = differential_lambda(W, p, diff)
    vis = chunk_mask(T, m["mask"]["size"])
    heads = []
    for a in range(H):
        g = a // (H // G)
        a1 = softmax_attention(q[:, a, 0], k[:, g, 0], v[:, g], vis, m["scale"])
        a2 = softmax_attention(q[:, a, 1], k[:, g, 1], v[:, g], vis, m["scale"])
        heads.append(rms_norm(a1 - lam * a2, eps) * (1.0 - diff))
    return np.stack(heads, 1).reshape(T, H * vdim) @ W[p + "o"].T


def poly_norm(z, coeff, eps):
    a, b, c, e = coeff
    return a * rms_norm(z, eps) + b * rms_norm(z ** 2, eps) + c * rms_norm(z ** 3, eps) + e


def dense_ff(h, W, p, eps):
    return poly_norm(h @ W[p + "up"].T, W[p + "act"], eps) @ W[p + "down"].T


def route_top(logits, top):
    """Per token: the `top` largest logits (ties: lowest index) and the softmax over those alone."""
    order = np.argsort(-logits, axis=-1, kind="stable")[:, :top]
    z = np.take_along_axis(logits, order, -1)
    w = np.exp(z - z.max(-1, keepdims=True))
    return order, w / w.sum(-1, keepdims=True)


def moe_ff(h, W, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ W[p + "router"].T + W[p + "router.b"]
    idx, wt = route_top(logits, top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            assert e < E
            g, u = W[p + f"e{e}.gate"] @ h[t], W[p + f"e{e}.up"] @ h[t]
            out[t] += wt[t, c] * (W[p + f"e{e}.down"] @ (g * sigmoid(g) * u))
    return out


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and, on request, the stream that leaves every layer, after the depth average)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    history = [x]
    kv_of = {}
    streams = []
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = token_shift(rms_norm(x, eps, W[p + "norm1"], True), W[p + "shift"])
        if L["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", m, eps)
        elif L["type"] == "latent_attention_2":
            y = latent_attention_2(h, W, p + "mix.", m, eps)
        elif L["type"] == "attention":
            if "kv_from" in m and m["kv_from"] is not None:
                kv = kv_of[m["kv_from"]]
            else:
                kv = kv_of[i] = keys_values(h, W, p + "mix.", m)
            y = differential_attention(h, W, p + "mix.", m, eps, kv)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, eps, W[p + "norm1b"], True)
        if L["mlp"] is not None:
            h = rms_norm(x, eps, W[p + "norm2"], True)
            y = dense_ff(h, W, p + "mlp.", eps) if L["mlp"]["kind"] == "dense" else moe_ff(h, W, p + "mlp.", L["mlp"])
            x = x + rms_norm(y, eps, W[p + "norm2b"], True)
        history.append(x)
        x = depth_average(history, W[p + "dwa"])
        streams.append(x)
    logits = rms_norm(x, eps, W["final.norm"], True) @ W["head"].T * cfg["logit_scale"]
    return (logits, np.stack(streams)) if return_layers else logits
