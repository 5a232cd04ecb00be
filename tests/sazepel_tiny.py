"""Small Sazepel configurations and weights for the tests.

The configurations differ from each other in every size and constant, and within one no two sizes that could be
confused are equal by accident (key and value sizes, head counts of the two mixers of a layer, widths).  Rotations
over part of a vector, over all of it and over none; decays of exactly 1 and well below; as many key/value heads as
heads, one for all heads, and groups in between; routers that choose 1 of 3, 2 of 4 and all 5 of 5 experts; expert
widths that are no multiples of 8; layers without a feed-forward; head sizes that take the tensor-core kernels in
bfloat16 (16, 32) and ones that do not (20, 24); a logit factor away from 1.  `TINY_R` has no routers, so that a
bfloat16 run can be compared at every position; `make_weights(..., decided=True)` makes routers whose biases decide the
choice (the same experts for every token, weights that still vary), for the same reason.

`make_weights` draws values that a bfloat16 holds exactly, so that the plain implementation, the 32-bit engine and
the bfloat16 engine read the same numbers.  Scales are chosen so that faults show: the layer norms' single numbers
away from 1, head-mixing matrices with entries of both signs and of order 1, router biases of the order of the
logits, the two side-by-side weights unequal.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def _ret(heads, dim, vdim, decay, base, dims):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": dims}}


def _att(heads, kv_heads, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


TINY_P = {
    "architecture": "Sazepel", "vocab": 101, "width": 40, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
    "layers": [
        {"type": "parallel", "mixer": {"left": _att(4, 2, 16, 24, 0.5), "right": _ret(3, 8, 12, (0.5, 0.9, 1.0), 100.0, 4)},
         "mlp": _moe(20, 4, 2)},
        {"type": "retention", "mixer": _ret(2, 16, 8, (0.97, 0.8), 10000.0, 16), "mlp": None},
        {"type": "parallel", "mixer": {"left": _att(3, 3, 20, 12, 0.6), "right": _ret(1, 12, 20, (0.93,), 50.0, 0)},
         "mlp": _moe(16, 3, 1)},
    ],
}

TINY_Q = {
    "architecture": "Sazepel", "vocab": 67, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "layers": [
        {"type": "retention", "mixer": _ret(1, 40, 36, (0.99,), 500.0, 20), "mlp": _moe(24, 5, 5)},
        {"type": "parallel", "mixer": {"left": _att(8, 1, 32, 16, 0.4), "right": _ret(2, 24, 28, (1.0, 0.75), 1000.0, 24)},
         "mlp": None},
        {"type": "retention", "mixer": _ret(4, 12, 16, (0.6, 0.9, 0.95, 0.999), 20.0, 8), "mlp": _moe(40, 2, 1)},
        {"type": "parallel", "mixer": {"left": _att(2, 2, 24, 40, 0.35), "right": _ret(2, 16, 16, (0.9, 0.98), 300.0, 16)},
         "mlp": _moe(8, 6, 3)},
    ],
}

TINY_R = {
    "architecture": "Sazepel", "vocab": 131, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
    "layers": [
        {"type": "parallel", "mixer": {"left": _att(6, 2, 32, 16, 0.45), "right": _ret(2, 32, 24, (0.9, 0.995), 10000.0, 32)},
         "mlp": None},
        {"type": "retention", "mixer": _ret(3, 16, 20, (0.7, 0.96, 0.99), 200.0, 12), "mlp": None},
        {"type": "parallel", "mixer": {"left": _att(4, 4, 16, 16, 0.7), "right": _ret(1, 64, 48, (0.98,), 1e6, 64)},
         "mlp": None},
    ],
}

TINY_S = {
    "architecture": "Sazepel", "vocab": 89, "width": 32, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
    "layers": [
        {"type": "retention", "mixer": _ret(2, 16, 16, (0.9375, 0.99), 1e4, 8), "mlp": _moe(24, 4, 2)},
        {"type": "parallel", "mixer": {"left": _att(4, 2, 16, 32, 0.3), "right": _ret(2, 8, 8, (0.8, 1.0), 100.0, 8)},
         "mlp": _moe(16, 5, 3)},
    ],
}

CONFIGS = {"p": TINY_P, "q": TINY_Q, "r": TINY_R, "s": TINY_S}


def bf16_exact(x):
    """Rounds float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    shape = np.shape(x)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(shape)


def _retention_shapes(p, mx, E):
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    return {f"{p}.q": (H * D, E), f"{p}.k": (H * D, E), f"{p}.v": (H * V, E), f"{p}.g": (H * V, E), f"{p}.o": (E, H * V)}


def tensor_shapes(config) -> dict:
    E, V = config["width"], config["vocab"]
    out = {"embed": (V, E), "embed.norm": (), "head": (V, E), "final.norm": ()}
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}", layer["mixer"]
        out[f"{p}.norm1"] = ()
        out[f"{p}.norm1b"] = ()
        if layer["type"] == "retention":
            out.update(_retention_shapes(f"{p}.mix", mx, E))
        else:
            lf = mx["left"]
            H, G, D, Vd = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            out.update({f"{p}.mix.left.q": (H * D, E), f"{p}.mix.left.k": (G * D, E), f"{p}.mix.left.v": (G * Vd, E),
                        f"{p}.mix.left.talk": (H, H), f"{p}.mix.left.g": (H * Vd, E), f"{p}.mix.left.o": (E, H * Vd),
                        f"{p}.mix.left.out": (E,), f"{p}.mix.right.out": (E,)})
            out.update(_retention_shapes(f"{p}.mix.right", mx["right"], E))
        mlp = layer["mlp"]
        if mlp is not None:
            F, n = mlp["expert"]["ff"], mlp["router"]["experts"]
            out.update({f"{p}.norm2": (), f"{p}.norm2b": (), f"{p}.mlp.router": (n, E), f"{p}.mlp.router.b": (n,)})
            for e in range(n):
                out.update({f"{p}.mlp.e{e}.gate": (F, E), f"{p}.mlp.e{e}.up": (F, E), f"{p}.mlp.e{e}.down": (E, F)})
    return out


def make_weights(config, seed: int, std: float = 0.1, decided: bool = False) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if shape == ():
            x = np.asarray(rng.uniform(0.6, 1.6))
        elif last == "out":
            x = 1.0 + rng.normal(0.0, 0.4, shape)
        elif last == "talk":
            x = np.eye(shape[0]) * 0.8 + rng.normal(0.0, 0.5, shape)
        elif last == "b":
            x = rng.permutation(shape[0]) * 4.0 if decided else rng.normal(0.0, 1.0, shape)
        elif last == "router":
            x = rng.normal(0.0, 0.05 if decided else 0.5, shape)
        elif name == "embed":
            x = rng.normal(0.0, 1.0, shape)
        else:
            x = rng.normal(0.0, std * (48.0 / shape[-1]) ** 0.5 * 1.5, shape)
            if last == "k" and ".left." not in name:
                # a retention's k leans towards its q, so that q . k of one token is seldom near zero (see
                # `sure_first_tokens`); tensor_shapes lists q before k
                x = 0.6 * out[name[:-1] + "q"] + 0.8 * x
        out[name] = bf16_exact(np.asarray(x, np.float32))
    return out


def sure_first_tokens(config, weights, floor: float = 0.04) -> list:
    """The tokens that can open a sequence in a test.  From an empty state a retention head's first output is
    (q . k) v, of which the head norm keeps the sign of q . k alone: a token whose q and k are nearly at right angles
    in some head of some layer gets one sign or the other by rounding (no fault, and not small).  These are the
    tokens for which |cos(q, k)| >= floor in every head, by the plain implementation."""
    import plain_sazepel
    out = []
    for t in range(config["vocab"]):
        cosines = []
        plain_sazepel.forward(config, weights, [t], cosines=cosines)
        if all((c >= floor).all() for c in cosines):
            out.append(t)
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


def random_config(seed: int) -> dict:
    """A configuration drawn from a fixed seed: 2 to 5 layers in any order, sizes of every kind."""
    rng = np.random.default_rng(1000 + seed)

    def pick(*xs):
        return xs[int(rng.integers(0, len(xs)))]

    def ret():
        heads, dim = pick(1, 2, 3, 5), pick(8, 12, 16, 20, 32, 64, 72)
        dims = pick(0, dim, dim // 2 if (dim // 2) % 2 == 0 else dim)
        decay = [float(pick(1.0, 0.5, 0.9, 0.97, 0.995, 1.0 - 2.0 ** -7)) for _ in range(heads)]
        return _ret(heads, dim, pick(8, 12, 16, 24, 40, 64), decay, float(pick(10.0, 1e4, 1e6)), dims)

    def att():
        kv = pick(1, 2, 3, 4)
        return _att(kv * pick(1, 2, 3), kv, pick(8, 16, 20, 32, 48, 64), pick(8, 16, 24, 32, 80), float(pick(0.2, 0.4, 0.6)))

    layers = []
    for _ in range(int(rng.integers(2, 6))):
        experts = pick(1, 2, 4, 7)
        mlp = pick(None, _moe(pick(8, 12, 24, 36), experts, int(rng.integers(1, experts + 1))))
        if rng.random() < 0.5:
            layers.append({"type": "retention", "mixer": ret(), "mlp": mlp})
        else:
            layers.append({"type": "parallel", "mixer": {"left": att(), "right": ret()}, "mlp": mlp})
    return {"architecture": "Sazepel", "vocab": pick(97, 150, 257), "width": pick(24, 37, 56, 64, 100),
            "norm": {"eps": float(pick(1e-6, 1e-5, 1e-3))}, "logit_scale": float(pick(0.25, 1.0, 2.0)), "layers": layers}
