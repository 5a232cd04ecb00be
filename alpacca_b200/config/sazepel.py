"""The configuration of the Sazepel decoder, by its config.json keys.

    {"architecture": "Sazepel", "vocab": V, "width": E, "norm": {"eps": e}, "logit_scale": s,
     "layers": [{"type": "retention" | "parallel", "mixer": {...}, "mlp": {...} | null}, ...]}

A layer's mixer sizes:
    retention   heads, dim, vdim, decay (one number per head, in (0, 1]), rot: {base, dims}
    parallel    left: {heads, kv_heads, dim, vdim, scale}      attention whose softmax weights are mixed across heads
                right: a retention's sizes
and its feed-forward: {"kind": "moe", "expert": {"ff": F}, "router": {"experts": n, "top": k}}.
Every size and constant is read from here; the configuration sets no limit on positions.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ModelConfig
from .lefatar import _check_keys, _is_int, _is_num

RETENTION = {"heads": int, "dim": int, "vdim": int, "rot": dict}
MIXED_ATTENTION = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float}


def _check_retention(where: str, mx, bad: list) -> None:
    if not _check_keys(where, mx, RETENTION, bad):
        return
    decay = mx.get("decay")
    if not (isinstance(decay, list) and len(decay) == mx["heads"] and all(_is_num(a) and 0 < a <= 1 for a in decay)):
        bad.append(f"{where}.decay must list one number in (0, 1] per head")
    rot = mx["rot"]
    if _check_keys(f"{where}.rot", rot, {"base": float}, bad):
        dims = rot.get("dims")
        if not (_is_int(dims) and dims >= 0 and dims % 2 == 0 and dims <= mx["dim"]):
            bad.append(f"{where}.rot.dims {dims!r} must be even and at most dim {mx['dim']} (0: no rotation)")
        if not rot["base"] > 0:
            bad.append(f"{where}.rot.base must be positive")


def _check_mixed_attention(where: str, mx, bad: list) -> None:
    if _check_keys(where, mx, MIXED_ATTENTION, bad) and mx["heads"] % mx["kv_heads"]:
        bad.append(f"{where}: {mx['heads']} heads cannot share {mx['kv_heads']} key/value heads")


@dataclass(frozen=True)
class SazepelConfig(ModelConfig):
    vocab: int = None
    width: int = None
    norm: dict = field(default_factory=dict)
    layers: list = field(default_factory=list)
    logit_scale: float = 1.0
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

    def validate(self) -> list[str]:
        bad: list[str] = []
        for name in ("vocab", "width"):
            v = getattr(self, name)
            if not (_is_int(v) and v > 0):
                bad.append(f"key '{name}' must be a positive integer, got {v!r}")
        if not (isinstance(self.norm, dict) and _is_num(self.norm.get("eps")) and self.norm["eps"] >= 0):
            bad.append("norm.eps must be a number that is not negative")
        if not _is_num(self.logit_scale):
            bad.append("logit_scale must be a number")
        if not isinstance(self.layers, list) or not self.layers:
            bad.append("'layers' must be a list with at least one layer")
            return bad
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                bad.append(f"{where} must be an object")
                continue
            kind = layer.get("type")
            if kind == "retention":
                _check_retention(f"{where}.mixer", layer.get("mixer"), bad)
            elif kind == "parallel":
                mx = layer.get("mixer")
                if _check_keys(f"{where}.mixer", mx, {"left": dict, "right": dict}, bad):
                    _check_mixed_attention(f"{where}.mixer.left", mx["left"], bad)
                    _check_retention(f"{where}.mixer.right", mx["right"], bad)
            else:
                bad.append(f"{where}.type {kind!r} is not supported (supported: parallel, retention)")
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
                if _check_keys(f"{where}.mlp.router", rt, {"experts": int, "top": int}, bad) and rt["top"] > rt["experts"]:
                    bad.append(f"{where}.mlp.router: {rt['top']} of {rt['experts']} experts cannot be chosen")
        for t in self.stop_tokens if not bad else ():
            if not 0 <= t < self.vocab:
                bad.append(f"eos_token_id {t} lies outside the vocabulary of {self.vocab}")
        return bad
