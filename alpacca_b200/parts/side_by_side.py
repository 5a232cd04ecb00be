"""Two mixers side by side: both read the same input, and the sub-layer's output is half the sum of their
outputs, each first divided by its root mean square over the model width and multiplied by a weight of its own:

    y = (unit(left(h)) * w_left + unit(right(h)) * w_right) / 2,     unit(v) = v / sqrt(mean(v^2) + eps)

Each mixer keeps what it keeps (keys and values, a state): a run of the block has one cache entry for each.  The sum
is not formed here: the block's kernel that adds a sub-layer's output to the float32 stream reads both outputs and
forms it on the way (`HalfSum`, `ops.post_norm_add`), so neither output makes a round trip of its own.
"""
from __future__ import annotations

from ..weights.loader import ParamSpec
from .base import BuildOptions, HalfSum, Mixer


class SideBySide(Mixer):
    def __init__(self, opts: BuildOptions, width: int, left: Mixer, right: Mixer, eps: float, prefix: str,
                 names=("left.out", "right.out")):
        self.opts, self.width, self.eps, self.prefix, self.names = opts, int(width), float(eps), prefix, names
        self.left, self.right = left, right
        self.w_left = self.w_right = None

    def own_param_specs(self):
        return [ParamSpec(f"{self.prefix}.{n}", (self.width,), "vector", "one_plus_normal") for n in self.names]

    def load_own(self, fetch):
        self.w_left, self.w_right = (fetch(s) for s in self.own_param_specs())

    def cache_specs(self) -> list:
        return [s for s in (self.left.cache_spec(), self.right.cache_spec()) if s is not None]

    def cache_spec(self):
        specs = self.cache_specs()
        if len(specs) > 1:
            raise ValueError(f"{self.prefix}: both mixers keep something; the block asks `cache_specs()`")
        return specs[0] if specs else None

    def forward(self, h, ctx, cache, write_cache: bool = True):
        views = list(cache) if isinstance(cache, (list, tuple)) else ([cache] if cache is not None else [])
        views = iter(views)
        left = self.left.forward(h, ctx, next(views) if self.left.cache_spec() is not None else None, write_cache)
        right = self.right.forward(h, ctx, next(views) if self.right.cache_spec() is not None else None, write_cache)
        if left.dtype != right.dtype:
            raise ValueError(f"{self.prefix}: the two mixers' outputs differ in dtype")
        return HalfSum(left, right, self.w_left, self.w_right, self.eps)
