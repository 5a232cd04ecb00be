"""The configuration of the Mavidra decoder, by its config.json keys.

    {"architecture": "Mavidra", "vocab": V, "width": E, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"scale": s, "bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "gla" | "latent_attention" | "parallel", "mixer": {...}, "mlp": {...} | null}, ...]}

A layer's mixer sizes:
    gla               heads, dim, vdim, tau; rank (the low-rank decay projection's inner size: where config.json leaves
                      it out it is read from the shape of the layer's tensor `mix.a1`, see `with_shapes`)
    latent_attention  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims}, mask: {size} (may be left
                      out: every earlier token is seen), kv_from: j (may be left out; the layer then has no
                      down-projection of its own and reads what layer j caches)
    parallel          left: {heads, kv_heads, dim, vdim, scale, rot: {base, dims}}      attention with a sink and a gate per head
                      right: {heads, kv_heads, dim, vdim, conv}                          the gated delta rule
                      left_scale, right_scale
and its feed-forward: {"kind": "moe", "expert": {"ff": F}, "router": {"experts": n, "top": k, "groups": {"count": g,
"keep": c}}} (groups may be left out: one group).  Every size and constant is read from here; the configuration sets
no limit on positions.
"""
from __future__ import annotations

import copy
import dataclasses
from dataclasses import dataclass, field

from .base import ModelConfig
from .lefatar import _check_keys, _is_int, _is_num

GLA = {"heads": int, "dim": int, "vdim": int, "tau": float}
LATENT = {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "q_rank": int, "kv_rank": int, "scale": float, "rot": dict}
LEFT = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "rot": dict}
RIGHT = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int}


def _check_rot(where: str, rot, limit: int, bad: list) -> None:
    if _check_keys(where, rot, {"base": float}, bad):
        dims = rot.get("dims")
        if not (_is_int(dims) and dims >= 0 and dims % 2 == 0 and dims <= limit):
            bad.append(f"{where}.dims {dims!r} must be even and at most {limit} (0: no rotation)")
        if not rot["base"] > 0:
            bad.append(f"{where}.base must be positive")


@dataclass(frozen=True)
class MavidraConfig(ModelConfig):
    vocab: int = None
    width: int = None
    norm: dict = field(default_factory=dict)
    embedding: dict = field(default_factory=dict)
    layers: list = field(default_factory=list)
    residual_mult: float = 1.0
    bos_token_id: int | None = None
    eos_token_id: int | list | None = None

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def stop_tokens(self) -> tuple[int, ...]:
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple)) else (int(e),)

    @property
    def bos_token(self) -> int | None:
        return self.bos_token_id

    def to_dict(self) -> dict:
        out = super().to_dict()
        out.pop("architectures", None)
        out = {"architecture": self.architecture, **out}
        for key in ("bos_token_id", "eos_token_id"):
            if out.get(key) is None:
                out.pop(key, None)
        return out

    def with_shapes(self, shapes: dict) -> "MavidraConfig":
        """The configuration with the sizes that only the checkpoint's tensors give: a gla layer's `rank` is the row
        count of its `mix.a1` where config.json does not name it."""
        layers = copy.deepcopy(self.layers)
        for i, layer in enumerate(layers):
            if isinstance(layer, dict) and layer.get("type") == "gla" and isinstance(layer.get("mixer"), dict):
                shape = shapes.get(f"l{i}.mix.a1")
                if "rank" not in layer["mixer"] and shape is not None and len(shape) == 2:
                    layer["mixer"]["rank"] = int(shape[0])
        return dataclasses.replace(self, layers=layers)

    def validate(self) -> list[str]:
        bad: list[str] = []
        for name in ("vocab", "width"):
            v = getattr(self, name)
            if not (_is_int(v) and v > 0):
                bad.append(f"key '{name}' must be a positive integer, got {v!r}")
        if not (isinstance(self.norm, dict) and _is_num(self.norm.get("eps")) and self.norm["eps"] >= 0):
            bad.append("norm.eps must be a number that is not negative")
        if not _is_num(self.residual_mult):
            bad.append("residual_mult must be a number")
        if _check_keys("embedding", self.embedding, {"scale": float}, bad) and self.embedding.get("bigram") is not None:
            _check_keys("embedding.bigram", self.embedding["bigram"], {"buckets": int, "mul_prev": int, "mul_cur": int}, bad)
        if not isinstance(self.layers, list) or not self.layers:
            bad.append("'layers' must be a list with at least one layer")
            return bad
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                bad.append(f"{where} must be an object")
                continue
            kind, mx = layer.get("type"), layer.get("mixer")
            if kind == "gla":
                if _check_keys(f"{where}.mixer", mx, GLA, bad):
                    if not mx["tau"] > 0:
                        bad.append(f"{where}.mixer.tau must be positive")
                    if "rank" in mx and not (_is_int(mx["rank"]) and mx["rank"] > 0):
                        bad.append(f"{where}.mixer.rank must be a positive integer")
            elif kind == "latent_attention":
                if _check_keys(f"{where}.mixer", mx, LATENT, bad):
                    _check_rot(f"{where}.mixer.rot", mx["rot"], mx["rot_dim"], bad)
                    mask = mx.get("mask")
                    if mask is not None:
                        _check_keys(f"{where}.mixer.mask", mask, {"size": int}, bad)
                    j = mx.get("kv_from")
                    if j is not None:
                        other = self.layers[j].get("mixer") if _is_int(j) and 0 <= j < i and \
                            isinstance(self.layers[j], dict) and self.layers[j].get("type") == "latent_attention" else None
                        if not isinstance(other, dict) or other.get("kv_from") is not None:
                            bad.append(f"{where}.mixer.kv_from {j!r} must name an earlier latent_attention layer that "
                                       "caches its own keys")
                        elif any(other.get(k) != mx.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                            bad.append(f"{where}.mixer: kv_rank, rot_dim and rot must equal those of layer {j}, whose "
                                       "cache it reads")
            elif kind == "parallel":
                if _check_keys(f"{where}.mixer", mx, {"left": dict, "right": dict, "left_scale": float,
                                                     "right_scale": float}, bad):
                    lf, rt = mx["left"], mx["right"]
                    if _check_keys(f"{where}.mixer.left", lf, LEFT, bad):
                        _check_rot(f"{where}.mixer.left.rot", lf["rot"], lf["dim"], bad)
                        if lf["heads"] % lf["kv_heads"]:
                            bad.append(f"{where}.mixer.left: {lf['heads']} heads cannot share {lf['kv_heads']} key/value heads")
                    if _check_keys(f"{where}.mixer.right", rt, RIGHT, bad) and rt["heads"] % rt["kv_heads"]:
                        bad.append(f"{where}.mixer.right: {rt['heads']} heads cannot share {rt['kv_heads']} query/key heads")
            else:
                bad.append(f"{where}.type {kind!r} is not supported (supported: gla, latent_attention, parallel)")
                continue
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                bad.append(f"{where}.mlp must be null or an object of kind 'moe'")
                continue
            if _check_keys(f"{where}.mlp", mlp, {"expert": dict, "router": dict}, bad):
                _check_keys(f"{where}.mlp.expert", mlp["expert"], {"ff": int}, bad)
                rt = mlp["router"]
                if _check_keys(f"{where}.mlp.router", rt, {"experts": int, "top": int}, bad):
                    E, G, keep = rt["experts"], 1, 1
                    if rt.get("groups") is not None:
                        if not _check_keys(f"{where}.mlp.router.groups", rt["groups"], {"count": int, "keep": int}, bad):
                            continue
                        G, keep = rt["groups"]["count"], rt["groups"]["keep"]
                    if E % G:
                        bad.append(f"{where}.mlp.router: {E} experts do not form {G} equal groups")
                    elif keep > G or rt["top"] > keep * (E // G):
                        bad.append(f"{where}.mlp.router: {rt['top']} experts cannot be chosen from {keep} of {G} "
                                   f"groups of {E // G}")
        for t in self.stop_tokens if not bad else ():
            if not 0 <= t < self.vocab:
                bad.append(f"eos_token_id {t} lies outside the vocabulary of {self.vocab}")
        return bad
