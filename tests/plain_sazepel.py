"""A plain, slow implementation of the Sazepel decoder in NumPy float64: whole sequences, no cache, no
batches, one function per mechanism.  It shares no code with the package; the tests hold the package to it.

A model is (config dict, {tensor name: array}).  Layer i's tensors are `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`,
`l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`; linear weights are [out, in].

    start:   x = unit(embed[token]) * embed.norm
    layer:   x <- x + unit(mixer(unit(x) * n1)) * n1b;   x <- x + unit(ff(unit(x) * n2)) * n2b  (if it has a ff)
    unit(x): x / sqrt(mean(x^2) + eps); a layer norm's weight is ONE number
    end:     logits = head (unit(x) * final.norm) * logit_scale
"""
from __future__ import annotations

import numpy as np


def unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def turn_halves(x, positions, rot):
    """x [T, heads, D]: of each head's first rot.dims numbers, number i and number i + dims/2 form a pair that is
    turned by the angle position * base^(-2i/dims); the other numbers stay."""
    dims = int(rot["dims"])
    out = np.array(x, dtype=np.float64, copy=True)
    if dims == 0:
        return out
    half = dims // 2
    freq = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def retention(h, w, mx, eps, positions=None, state=None, cosines=None):
    """Linear attention with a constant decay per head.  h [T, E]; returns ([T, E], final state [H, D, V]).
    `cosines`: a list that gets, per head, |cos| of the angle between the first token's q and k: from an empty state
    that token's output is (q . k) v, so that after the head norm only the SIGN of q . k is left."""
    T = h.shape[0]
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    positions = np.arange(T) if positions is None else positions
    q = turn_halves((h @ w["q"].T).reshape(T, H, D), positions, mx["rot"])
    k = turn_halves((h @ w["k"].T).reshape(T, H, D), positions, mx["rot"]) * D ** -0.5
    v = (h @ w["v"].T).reshape(T, H, V)
    S = np.zeros((H, D, V)) if state is None else np.array(state, np.float64)
    if cosines is not None:
        cosines.append(np.abs((q[0] * k[0]).sum(-1)) / (np.linalg.norm(q[0], axis=-1) * np.linalg.norm(k[0], axis=-1) + 1e-300))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            S[a] = mx["decay"][a] * S[a] + np.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    o = unit(o, eps).reshape(T, H * V) * silu(h @ w["g"].T)
    return o @ w["o"].T, S


def talking_attention(h, w, mx, eps):
    """Causal softmax attention without positions whose softmax weights are mixed across heads before they
    meet the values.  h [T, E] -> [T, E]."""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    per = H // G
    q = unit((h @ w["q"].T).reshape(T, H, D), eps)
    k = unit((h @ w["k"].T).reshape(T, G, D), eps)
    v = unit((h @ w["v"].T).reshape(T, G, V), eps)
    P = np.zeros((H, T, T))
    seen = np.tril(np.ones((T, T), bool))
    for a in range(H):
        s = (q[:, a] @ k[:, a // per].T) * mx["scale"]
        s = np.where(seen, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        P[a] = e / e.sum(axis=1, keepdims=True)
    mixed = np.einsum("ab,bij->aij", w["talk"], P)
    o = np.stack([mixed[a] @ v[:, a // per] for a in range(H)], axis=1).reshape(T, H * V)
    o = o * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def side_by_side(h, w, mx, eps, positions=None, cosines=None):
    left = talking_attention(h, _sub(w, "left."), mx["left"], eps)
    right, _ = retention(h, _sub(w, "right."), mx["right"], eps, positions, cosines=cosines)
    return 0.5 * (unit(left, eps) * w["left.out"] + unit(right, eps) * w["right.out"])


def route(h, w, router):
    """(experts [T, top], weights [T, top]): the experts with the largest logits and the softmax over just those."""
    z = h @ w["router"].T + w["router.b"]
    top = router["top"]
    chosen = np.argsort(-z, axis=1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=1)
    e = np.exp(zc - zc.max(axis=1, keepdims=True))
    return chosen, e / e.sum(axis=1, keepdims=True), z


def experts(h, w, mlp, margins=None):
    chosen, wts, z = route(h, w, mlp["router"])
    if margins is not None:      # per token: how far the last chosen logit lies above the first one left out
        zs = -np.sort(-z, axis=1)
        top = mlp["router"]["top"]
        margins.append(zs[:, top - 1] - zs[:, top] if top < z.shape[1] else np.full(z.shape[0], np.inf))
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(chosen[t]):
            a = silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])
            out[t] += wts[t, j] * (w[f"e{e}.down"] @ a)
    return out


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, trace=None, margins=None, cosines=None):
    """Logits [T, vocab] of the whole sequence `tokens`.  `trace`: a list that gets the stream after every layer;
    `margins`: a list that gets, for every router, each token's gap between the last chosen logit and the next;
    `cosines`: a list that gets, for every retention, what `retention` says of the first token."""
    W = {k: np.asarray(v, np.float64) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = unit(W["embed"][np.asarray(tokens)], eps) * W["embed.norm"]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = unit(x, eps) * W[p + "norm1"]
        mix = _sub(W, p + "mix.")
        if layer["type"] == "retention":
            y, _ = retention(h, mix, layer["mixer"], eps, cosines=cosines)
        elif layer["type"] == "parallel":
            y = side_by_side(h, mix, layer["mixer"], eps, cosines=cosines)
        else:
            raise ValueError(layer["type"])
        x = x + unit(y, eps) * W[p + "norm1b"]
        if layer.get("mlp") is not None:
            h = unit(x, eps) * W[p + "norm2"]
            x = x + unit(experts(h, _sub(W, p + "mlp."), layer["mlp"], margins), eps) * W[p + "norm2b"]
        if trace is not None:
            trace.append(x.copy())
    return (unit(x, eps) * W["final.norm"]) @ W["head"].T * float(config["logit_scale"])
