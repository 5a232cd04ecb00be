"""Two mixers side by side: both read the same input, and the sub-layer's output is half the sum of their
outputs, each first divided by its root mean square over the model width and multiplied by a weight of its own:

    y = (unit(left(h)) * w_left + unit(right(h)) * w_right) / 2,     unit(v) = v / sqrt(mean(v^2) + eps)

or, with `scales=(c_left, c_right)`, the plain weighted sum y = c_left * left(h) + c_right * right(h) (no norms, no
tensors of its own; a `WeightedSum`).

Each mixer keeps what it keeps (keys and values, a state): a run of the block has one cache entry for each.  The sum
is not formed here: the block's kernel that adds a sub-layer's output to the float32 stream reads both outputs and
forms it on the way (`HalfSum`, `ops.post_norm_add`), so neither output makes a round trip of its own.
"""
from __future__ import annotations

from ..weights.loader import ParamSpec
from .base import BuildOptions, HalfSum, Mixer, WeightedSum, mixer_cache_specs


class SideBySide(Mixer):
    def __init__(self, opts: BuildOptions, width: int, left: Mixer, right: Mixer, eps: float, prefix: str,
                 names=("left.out", "right.out"), scales=None):
        self.opts, self.width, self.eps, self.prefix, self.names = opts, int(width), float(eps), prefix, names
        self.left, self.right = left, right
        self.w_left = self.w_right = None
        self.scales = None if scales is None else (float(scales[0]), float(scales[1]))

    def own_param_specs(self):
        if self.scales is not None:
            return []
        return [ParamSpec(f"{self.prefix}.{n}", (self.width,), "vector", "one_plus_normal") for n in self.names]

    def load_own(self, fetch):
        if self.scales is None:
            self.w_left, self.w_right = (fetch(s) for s in self.own_param_specs())

    def cache_specs(self) -> list:
        return mixer_cache_specs(self.left) + mixer_cache_specs(self.right)

    def cache_spec(self):
        specs = self.cache_specs()
        if len(specs) > 1:
            raise ValueError(f"{self.prefix}: both mixers keep something; the block asks `cache_specs()`")
        return specs[0] if specs else None

    def forward(self, h, ctx, cache, write_cache: bool = True):
        views = list(cache) if isinstance(cache, (list, tuple)) else ([cache] if cache is not None else [])
        n_left = len(mixer_cache_specs(self.left))

        def share(part):          # one view as it is, several as a list, none as None
            return part[0] if len(part) == 1 else (part or None)
        left = self.left.forward(h, ctx, share(views[:n_left]), write_cache)
        right = self.right.forward(h, ctx, share(views[n_left:]), write_cache)
        if left.dtype != right.dtype:
            raise ValueError(f"{self.prefix}: the two mixers' outputs differ in dtype")
        if self.scales is not None:
            return WeightedSum(left, right, *self.scales)
        return HalfSum(left, right, self.w_left, self.w_right, self.eps)
