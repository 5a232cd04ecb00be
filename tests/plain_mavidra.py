"""A plain, slow implementation of the Mavidra decoder in NumPy float64: whole sequences, no cache, no batches,
one function per mechanism.  It shares no code with the package; the tests hold the package to it.

A model is (config dict, {tensor name: array}).  Layer i's tensors are `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`,
`l<i>.norm2b` (each with a bias `<name>.b`), `l<i>.mix.*`, `l<i>.mlp.*`; linear weights are [out, in].

    start:   x = embed[token] * scale + bigram[(prev * mul_prev + token * mul_cur) mod buckets]   (row `buckets` for
             a sequence's first token)
    layer:   x <- x + m * LN1b(mixer(LN1(x)));   x <- x + m * LN2b(ff(LN2(x)))  (if it has a ff)
    LN(x):   (x - mean) / sqrt(var + eps) * w + b
    end:     logits = embed LN_final(x)
"""
from __future__ import annotations

import numpy as np


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    d = x - mu
    return d / np.sqrt((d * d).mean(axis=-1, keepdims=True) + eps) * w + b


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def embed(tokens, W, emb):
    """[T, E]: the scaled token rows plus the rows of the hashed table of (previous token, token) pairs."""
    tokens = np.asarray(tokens, np.int64)
    x = W["embed"][tokens] * float(emb["scale"])
    bg = emb.get("bigram")
    if bg is not None:
        rows = np.empty(len(tokens), np.int64)
        rows[0] = bg["buckets"]
        rows[1:] = (tokens[:-1] * bg["mul_prev"] + tokens[1:] * bg["mul_cur"]) % bg["buckets"]
        x = x + W["bigram"][rows]
    return x


def turn(x, positions, rot, interleaved):
    """x [T, heads, D]: the first rot.dims numbers of each head are turned pair by pair by position * base^(-2i/dims);
    pair i is (i, i + dims/2), or, interleaved, (2i, 2i + 1)."""
    dims = int(rot["dims"])
    out = np.array(x, dtype=np.float64, copy=True)
    if dims == 0:
        return out
    half = dims // 2
    freq = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, window=None, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]; token i sees j <= i (with a window: i - j < window);
    `sink` [H]: exp(sink) joins each denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen &= (i - j) < window
    out = np.zeros((T, H, v.shape[-1]))
    for a in range(H):
        s = (q[:, a] @ k[:, a // per].T) * scale
        s = np.where(seen, s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        if sink is not None:
            m = np.maximum(m, sink[a])
        e = np.exp(s - m)
        den = e.sum(axis=1, keepdims=True)
        if sink is not None:
            den = den + np.exp(sink[a] - m)
        out[:, a] = (e / den) @ v[:, a // per]
    return out


def gated_attention(h, w, mx, eps):
    """The left mixer of a parallel layer: grouped heads, query/key norm, rotation in halves, sink, a gate per head."""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T)
    q = rms((h @ w["q"].T).reshape(T, H, D), eps) * w["q.norm"]
    k = rms((h @ w["k"].T).reshape(T, G, D), eps) * w["k.norm"]
    v = (h @ w["v"].T).reshape(T, G, V)
    q, k = turn(q, pos, mx["rot"], False), turn(k, pos, mx["rot"], False)
    o = softmax_attention(q, k, v, float(mx["scale"]), None, w["sink"])
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w["o"].T


def short_conv(x, taps):
    """x [T, C], taps [C, K] (the last column is the current token's); zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    y = np.zeros_like(x)
    for j in range(K):
        back = K - 1 - j
        if back < T:
            y[back:] += x[:T - back] * taps[:, j]
    return y


def gated_delta_rule(h, w, mx, eps):
    """The right mixer of a parallel layer."""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    per = H // G
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)
    g = np.exp(-np.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    S = np.zeros((H, D, V))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            kk, qq = k[t, a // per], q[t, a // per]
            S[a] = g[t, a] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ kk)
            S[a] = S[a] + np.outer(kk, u)
            o[t, a] = S[a].T @ qq
    o = rms(o, eps) * w["norm"]
    o = o.reshape(T, H * V) * silu(h @ w["g"].T)
    return o @ w["o"].T


def parallel(h, w, mx, eps):
    left = gated_attention(h, _sub(w, "left."), mx["left"], eps)
    right = gated_delta_rule(h, _sub(w, "right."), mx["right"], eps)
    return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right


def gla(h, w, mx, eps):
    """Gated linear attention: a decay per key channel and token."""
    T = h.shape[0]
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    q = (h @ w["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).reshape(T, H, D)
    v = (h @ w["v"].T).reshape(T, H, V)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / float(mx["tau"]))).reshape(T, H, D)
    S = np.zeros((H, D, V))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            S[a] = alpha[t, a][:, None] * S[a] + np.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    o = rms(o, eps) * w["norm"]
    o = o.reshape(T, H * V) * silu(h @ w["g"].T)
    return o @ w["o"].T


def latent_keys(h, w, mx, eps):
    """What a latent-attention layer caches: (c [T, kv_rank], the turned key part [T, rot_dim])."""
    C, R = mx["kv_rank"], mx["rot_dim"]
    d = h @ w["dkv"].T
    c = rms(d[:, :C], eps) * w["dkv.norm"]
    r = turn(d[:, None, C:C + R], np.arange(h.shape[0]), mx["rot"], True)[:, 0]
    return c, r


def latent_attention(h, w, mx, eps, kept):
    """`kept`: (c, r) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, D, R, V = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    c, r = kept
    cq = rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(T, H, D + R)
    q_rot = turn(q[:, :, D:], np.arange(T), mx["rot"], True)
    k = np.concatenate([(c @ w["uk"].T).reshape(T, H, D), np.repeat(r[:, None, :], H, axis=1)], axis=-1)
    v = (c @ w["uv"].T).reshape(T, H, V)
    qq = np.concatenate([q[:, :, :D], q_rot], axis=-1)
    window = mx.get("mask", {}).get("size") if mx.get("mask") else None
    o = softmax_attention(qq, k, v, float(mx["scale"]), window)
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w["o"].T


def route(h, w, router):
    """(experts [T, top], weights [T, top], margin [T]): sigmoid scores; the choice adds a correction and is limited to
    the best groups (a group's score: its two largest choice scores); the weights are the plain scores."""
    s = sigmoid(h @ w["router"].T)
    choice = s + w["correction"]
    T, E = s.shape
    top = router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    n, keep = groups["count"], groups["keep"]
    per = E // n
    masked = choice.copy()
    margin = np.full(T, np.inf)
    if keep < n:
        gs = np.sort(choice.reshape(T, n, per), axis=2)[:, :, -2:].sum(axis=2)
        order = np.argsort(-gs, axis=1, kind="stable")
        gsorted = np.take_along_axis(gs, order, axis=1)
        margin = gsorted[:, keep - 1] - gsorted[:, keep]
        for t in range(T):
            for g in order[t, keep:]:
                masked[t, g * per:(g + 1) * per] = -np.inf
    chosen = np.argsort(-masked, axis=1, kind="stable")[:, :top]
    ms = -np.sort(-masked, axis=1)
    if top < E:
        with np.errstate(invalid="ignore"):
            gap = ms[:, top - 1] - ms[:, top]
        margin = np.minimum(margin, np.where(np.isnan(gap), np.inf, gap))
    return chosen, np.take_along_axis(s, chosen, axis=1), margin


def experts(h, w, mlp, margins=None):
    chosen, wts, margin = route(h, w, mlp["router"])
    if margins is not None:
        margins.append(margin)
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(chosen[t]):
            a = silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])
            out[t] += wts[t, j] * (w[f"e{e}.down"] @ a)
    return out


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, trace=None, margins=None):
    """Logits [T, vocab] of the whole sequence `tokens`.  `trace`: a list that gets the stream after every layer;
    `margins`: a list that gets, for every router, each token's distance from another choice."""
    W = {k: np.asarray(v, np.float64) for k, v in weights.items()}
    eps, m = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    x = embed(tokens, W, config["embedding"])
    kept = {}

    def ln(name, v):
        return layer_norm(v, W[name], W[name + ".b"], eps)

    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = ln(p + "norm1", x)
        mix, mx = _sub(W, p + "mix."), layer["mixer"]
        if layer["type"] == "gla":
            y = gla(h, mix, mx, eps)
        elif layer["type"] == "parallel":
            y = parallel(h, mix, mx, eps)
        elif layer["type"] == "latent_attention":
            if mx.get("kv_from") is None:
                kept[i] = latent_keys(h, mix, mx, eps)
            y = latent_attention(h, mix, mx, eps, kept[i if mx.get("kv_from") is None else mx["kv_from"]])
        else:
            raise ValueError(layer["type"])
        x = x + m * ln(p + "norm1b", y)
        if layer.get("mlp") is not None:
            h = ln(p + "norm2", x)
            x = x + m * ln(p + "norm2b", experts(h, _sub(W, p + "mlp."), layer["mlp"], margins))
        if trace is not None:
            trace.append(x.copy())
    return ln("final.norm", x) @ W["embed"].T
