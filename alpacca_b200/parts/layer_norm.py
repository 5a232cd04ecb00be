"""Layer norm with a weight and a bias per column, fused with the residual add that precedes it.

    y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b

eps is inside the root; the variance is taken about the mean.  32-bit arithmetic on the float32 stream
(csrc/layer_norm.cu).  The checkpoint names the weight `<name><weight_suffix>` and the bias `<name><bias_suffix>`.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Norm


class LayerNorm(Norm):
    def __init__(self, opts: BuildOptions, width: int, eps: float, name: str, weight_suffix: str = ".weight",
                 bias_suffix: str = ".bias"):
        self.opts, self.width, self.eps, self.name = opts, int(width), float(eps), name
        self.weight_suffix, self.bias_suffix = weight_suffix, bias_suffix
        self.weight = self.bias = None

    def own_param_specs(self):
        return [ParamSpec(f"{self.name}{self.weight_suffix}", (self.width,), "vector", "one_plus_normal"),
                ParamSpec(f"{self.name}{self.bias_suffix}", (self.width,), "vector", "normal")]

    def load_own(self, fetch):
        self.weight, self.bias = (fetch(s) for s in self.own_param_specs())

    def forward(self, residual, delta, out=None, rows=None, n_rows=None):
        if out is None:
            n = (rows.numel() if rows is not None else residual.shape[0]) if n_rows is None else n_rows
            out = torch.empty((max(n, 0) if rows is not None else residual.shape[0], self.width),
                              dtype=self.opts.dtype, device=residual.device)
        return ops.layer_norm(residual, delta, self.weight, self.bias, self.eps, out, rows=rows, n_rows=n_rows)
