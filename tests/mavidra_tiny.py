"""Small Mavidra configurations and weights for the tests.

The configurations differ from each other in every size and constant, and within one no two sizes that could be
confused are equal by accident (key and value sizes, head counts of the two mixers of a layer, ranks, widths).
Windows of 5 to 130 tokens, shorter than a page, longer than a page, and, for a layer that reads another layer's
latent rows, smaller AND larger than the window of the layer that caches them; rotations over part, all and none of
a vector; convolutions over 1 to 5 tokens; as many key/value heads as heads, one for all, groups in between; routers
with 1 to 4 groups of which some or all are kept, groups of one expert (whose score is that one expert's); layers
without a feed-forward; multipliers and hash sizes of the pair table that are not those of any other; head sizes that
take the tensor-core kernels in bfloat16 and ones that do not.

`make_weights` draws values that a bfloat16 holds exactly, so that the plain implementation, the 32-bit engine and
the bfloat16 engine read the same numbers.  Scales are chosen so that faults show: norm weights away from 1 and
biases away from 0, sinks of the order of the scores, corrections of the order of the scores (some far below zero, so
that a choice score is negative), decays spread over (0, 1).  `decided=True` makes routers whose corrections decide
the choice (the same experts for every token, weights that still vary), so that a bfloat16 run can be compared at
every position.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def _gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims, window=None, kv_from=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
          "scale": scale, "rot": {"base": base, "dims": dims}}
    if window is not None:
        mx["mask"] = {"size": window}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return mx


def _par(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def _att(heads, kv_heads, dim, vdim, scale, base, dims):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": dims}}


def _gdr(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(ff, experts, top, count=None, keep=None):
    router = {"experts": experts, "top": top}
    if count is not None:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _emb(scale, buckets, mul_prev, mul_cur):
    return {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


TINY_A = {
    "architecture": "Mavidra", "vocab": 101, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "embedding": _emb(3.0, 53, 31, 7),
    "layers": [
        {"type": "latent_attention", "mixer": _lat(3, 16, 8, 12, 24, 20, 0.3, 100.0, 8, window=70), "mlp": _moe(20, 6, 2, 3, 2)},
        {"type": "gla", "mixer": _gla(2, 12, 20, 4.0, 5), "mlp": None},
        {"type": "parallel", "mixer": _par(_att(4, 2, 16, 24, 0.4, 1e4, 8), _gdr(6, 3, 8, 12, 3), 1.3, 0.6), "mlp": _moe(16, 4, 1, 2, 1)},
        {"type": "latent_attention", "mixer": _lat(2, 8, 8, 20, 12, 20, 0.5, 100.0, 8, window=33, kv_from=0), "mlp": None},
    ],
}

TINY_B = {
    "architecture": "Mavidra", "vocab": 67, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "embedding": _emb(0.5, 211, 5, 13),
    "layers": [
        {"type": "gla", "mixer": _gla(1, 40, 36, 16.0, 9), "mlp": _moe(24, 5, 5)},
        {"type": "parallel", "mixer": _par(_att(6, 1, 32, 16, 0.25, 5e5, 32), _gdr(2, 2, 24, 28, 1), 0.5, 1.5), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(4, 24, 4, 16, 20, 28, 0.2, 50.0, 4, window=5), "mlp": _moe(40, 8, 3, 4, 3)},
        {"type": "latent_attention", "mixer": _lat(5, 12, 4, 8, 16, 28, 0.35, 50.0, 4, window=130, kv_from=2), "mlp": _moe(8, 6, 3, 6, 4)},
        {"type": "gla", "mixer": _gla(4, 16, 8, 1.0, 3), "mlp": _moe(12, 2, 1, 2, 2)},
    ],
}

# no routers: a bfloat16 run can be compared at every position whatever the weights
TINY_C = {
    "architecture": "Mavidra", "vocab": 131, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.25,
    "embedding": _emb(8.0, 17, 1, 3),
    "layers": [
        {"type": "parallel", "mixer": _par(_att(6, 3, 32, 48, 0.2, 100.0, 0), _gdr(4, 1, 32, 16, 5), 1.0, 1.0), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(4, 32, 16, 32, 24, 48, 0.15, 1e4, 16), "mlp": None},
        {"type": "gla", "mixer": _gla(3, 64, 16, 8.0, 16), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(2, 16, 16, 16, 12, 48, 0.3, 1e4, 16, window=64, kv_from=1), "mlp": None},
    ],
}

CONFIGS = {"a": TINY_A, "b": TINY_B, "c": TINY_C}


def bf16_exact(x):
    """Rounds float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    shape = np.shape(x)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(shape)


def _norm_shapes(name, E):
    return {name: (E,), name + ".b": (E,)}


def tensor_shapes(config) -> dict:
    E, V = config["width"], config["vocab"]
    out = {"embed": (V, E), **_norm_shapes("final.norm", E)}
    if config["embedding"].get("bigram"):
        out["bigram"] = (config["embedding"]["bigram"]["buckets"] + 1, E)
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}", layer["mixer"]
        out.update(_norm_shapes(f"{p}.norm1", E))
        out.update(_norm_shapes(f"{p}.norm1b", E))
        m = f"{p}.mix"
        if layer["type"] == "gla":
            H, D, Vd, r = mx["heads"], mx["dim"], mx["vdim"], mx["rank"]
            out.update({f"{m}.q": (H * D, E), f"{m}.k": (H * D, E), f"{m}.v": (H * Vd, E), f"{m}.g": (H * Vd, E),
                        f"{m}.o": (E, H * Vd), f"{m}.norm": (Vd,), f"{m}.a1": (r, E), f"{m}.a2": (H * D, r),
                        f"{m}.a2.b": (H * D,)})
        elif layer["type"] == "latent_attention":
            H, D, R, Vd, Q, C = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["q_rank"], mx["kv_rank"]
            out.update({f"{m}.dq": (Q, E), f"{m}.dq.norm": (Q,), f"{m}.uq": (H * (D + R), Q), f"{m}.uk": (H * D, C),
                        f"{m}.uv": (H * Vd, C), f"{m}.g": (H, E), f"{m}.o": (E, H * Vd)})
            if mx.get("kv_from") is None:
                out.update({f"{m}.dkv": (C + R, E), f"{m}.dkv.norm": (C,)})
        else:
            lf, rt = mx["left"], mx["right"]
            H, G, D, Vd = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            a = f"{m}.left"
            out.update({f"{a}.q": (H * D, E), f"{a}.k": (G * D, E), f"{a}.v": (G * Vd, E), f"{a}.q.norm": (D,),
                        f"{a}.k.norm": (D,), f"{a}.sink": (H,), f"{a}.g": (H, E), f"{a}.o": (E, H * Vd)})
            H, G, D, Vd, K = rt["heads"], rt["kv_heads"], rt["dim"], rt["vdim"], rt["conv"]
            b = f"{m}.right"
            out.update({f"{b}.q": (G * D, E), f"{b}.q.conv": (G * D, K), f"{b}.k": (G * D, E), f"{b}.k.conv": (G * D, K),
                        f"{b}.v": (H * Vd, E), f"{b}.v.conv": (H * Vd, K), f"{b}.b": (H, E), f"{b}.A_log": (H,),
                        f"{b}.norm": (Vd,), f"{b}.a": (H, E), f"{b}.dt_bias": (H,), f"{b}.g": (H * Vd, E),
                        f"{b}.o": (E, H * Vd)})
        mlp = layer["mlp"]
        if mlp is not None:
            F, n = mlp["expert"]["ff"], mlp["router"]["experts"]
            out.update(_norm_shapes(f"{p}.norm2", E))
            out.update(_norm_shapes(f"{p}.norm2b", E))
            out.update({f"{p}.mlp.router": (n, E), f"{p}.mlp.correction": (n,)})
            for e in range(n):
                out.update({f"{p}.mlp.e{e}.gate": (F, E), f"{p}.mlp.e{e}.up": (F, E), f"{p}.mlp.e{e}.down": (E, F)})
    return out


def make_weights(config, seed: int, std: float = 0.1, decided: bool = False) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        two = ".".join(name.rsplit(".", 2)[-2:])
        if name in ("embed", "bigram"):
            x = rng.normal(0.0, 1.0, shape)
        elif two in ("norm1.b", "norm1b.b", "norm2.b", "norm2b.b", "norm.b"):
            x = rng.normal(0.0, 0.2, shape)
        elif two == "a2.b":
            x = rng.normal(1.5, 1.5, shape)                 # decays from about 0.5^(1/tau) to nearly 1
        elif last in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            x = rng.uniform(0.6, 1.6, shape)
        elif last == "norm":
            x = 1.0 + rng.normal(0.0, 0.3, shape)
        elif last == "sink":
            x = rng.normal(0.0, 1.5, shape)
        elif last == "A_log":
            x = rng.uniform(-2.0, 1.0, shape)
        elif last == "dt_bias":
            x = rng.normal(0.0, 1.0, shape)
        elif last == "conv":
            x = rng.normal(0.0, 0.6, shape)
        elif last == "correction":
            x = rng.permutation(shape[0]) * 4.0 - 6.0 if decided else rng.normal(-0.3, 0.6, shape)
        elif last == "router":
            x = rng.normal(0.0, 0.05 if decided else 0.5, shape)
        elif last == "a2":
            x = rng.normal(0.0, 0.5, shape)
        else:
            x = rng.normal(0.0, std * (48.0 / shape[-1]) ** 0.5 * 1.5, shape)
            if last == "k" and name.endswith("mix.k"):
                # a gla layer's k leans towards its q, so that q . k of a sequence's first token is seldom near zero:
                # from an empty state that token's output is (q . k) v, of which the head norm keeps the sign alone
                x = 0.6 * out[name[:-1] + "q"] + 0.8 * x
        out[name] = bf16_exact(np.asarray(x, np.float32))
    return out


def write_model_dir(path, config, weights) -> Path:
    """config.json + model.safetensors (bfloat16), through the package's writer."""
    import torch
    from alpacca_b200.weights import write_safetensors
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config))
    entries = [(n, "BF16", tuple(w.shape), (lambda w=w: torch.from_numpy(np.array(w)).to(torch.bfloat16)))
               for n, w in weights.items()]
    write_safetensors(path / "model.safetensors", entries)
    return path


def random_config(seed: int, routers: bool = True) -> dict:
    """A configuration drawn from a fixed seed: 2 to 6 layers in any order, sizes of every kind."""
    rng = np.random.default_rng(7000 + seed)

    def pick(*xs):
        return xs[int(rng.integers(0, len(xs)))]

    def moe():
        if not routers or rng.random() < 0.3:
            return None
        count = pick(1, 1, 2, 3, 4)
        per = pick(1, 2, 3, 5)
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, keep * per + 1))
        return _moe(pick(8, 12, 24, 36), count * per, top, *((count, keep) if count > 1 or rng.random() < 0.5 else ()))

    def rot(limit):
        dims = pick(0, limit, limit // 2 if (limit // 2) % 2 == 0 else limit)
        return float(pick(10.0, 1e4, 1e6)), dims

    layers, latents = [], []
    for i in range(int(rng.integers(2, 7))):
        kind = pick("gla", "latent_attention", "parallel")
        if kind == "gla":
            mx = _gla(pick(1, 2, 3, 5), pick(8, 12, 16, 20, 32, 64, 72, 136), pick(8, 12, 16, 24, 40, 64),
                      float(pick(1.0, 2.0, 16.0)), pick(1, 4, 7, 16))
        elif kind == "latent_attention":
            window = pick(None, 3, 17, 64, 65, 100)
            if latents and rng.random() < 0.5:
                j = pick(*latents)
                o = layers[j]["mixer"]
                mx = _lat(pick(1, 2, 5), pick(8, 16, 24), o["rot_dim"], pick(8, 16, 40), pick(8, 20), o["kv_rank"],
                          float(pick(0.2, 0.4)), o["rot"]["base"], o["rot"]["dims"], window, kv_from=j)
            else:
                R = pick(2, 4, 8, 16)
                base, dims = rot(R)
                # rot.dims = rot_dim in this design (0: the part is there and is not rotated)
                mx = _lat(pick(1, 2, 3, 6), pick(8, 16, 20, 32), R, pick(8, 16, 24, 48), pick(8, 12, 32),
                          pick(14, 24, 32, 48) if R != 2 else pick(14, 30), float(pick(0.15, 0.3, 0.5)), base,
                          R if dims else 0, window)
                latents.append(i)
        else:
            kv, dim = pick(1, 2, 3), pick(8, 16, 20, 32, 64)
            base, dims = rot(dim)
            g = pick(1, 2, 3)
            mx = _par(_att(kv * pick(1, 2, 3), kv, dim, pick(8, 16, 24, 32, 80), float(pick(0.2, 0.4, 0.6)), base, dims),
                      _gdr(g * pick(1, 2), g, pick(8, 16, 24, 40, 64, 130), pick(8, 12, 32, 48), pick(1, 2, 3, 4, 6)),
                      float(pick(0.5, 1.0, 1.2)), float(pick(0.7, 1.0, 1.1)))
        layers.append({"type": kind, "mixer": mx, "mlp": moe()})
    return {"architecture": "Mavidra", "vocab": pick(97, 150, 257), "width": pick(24, 37, 56, 64, 100),
            "norm": {"eps": float(pick(1e-6, 1e-5, 1e-3))}, "residual_mult": float(pick(0.3, 0.5, 1.0)),
            "embedding": _emb(float(pick(1.0, 4.0, 12.0)), pick(7, 61, 509), pick(1, 29, 1000003), pick(2, 11, 131)),
            "layers": layers}
