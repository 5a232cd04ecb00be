"""RMSNorm, fused with the residual add that precedes it.

inv = 1/sqrt(mean(x^2) + eps); y = (x * inv) * w  (alpacca/tensor.py:163-173);
eps is inside the root.  The weight multiplies as it is, or, with `unit_offset`
(checkpoints that keep w = weight - 1), as 1 + w: the sum is formed once, in
float32, when the weight is loaded.  With `scalar` the checkpoint keeps ONE number
for all columns (a tensor without dimensions); it is spread over the width when it
is loaded, so every kernel that takes a weight per column serves it.  `scale`
multiplies the weight once at load (a constant factor on what reads the norm, such
as a factor on the logits after the last norm).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Norm


class RMSNorm(Norm):
    def __init__(self, opts: BuildOptions, width: int, eps: float, name: str, weight_suffix: str = ".weight",
                 unit_offset: bool = False, scalar: bool = False, scale: float = 1.0):
        self.opts, self.width, self.eps, self.name = opts, int(width), float(eps), name
        self.weight_suffix, self.unit_offset = weight_suffix, bool(unit_offset)
        self.scalar, self.scale = bool(scalar), float(scale)
        self.weight = None

    def own_param_specs(self):
        return [ParamSpec(f"{self.name}{self.weight_suffix}", () if self.scalar else (self.width,), "vector",
                          "normal" if self.unit_offset else "one_plus_normal")]

    def load_own(self, fetch):
        self.weight = fetch(self.own_param_specs()[0])
        if self.scalar:
            self.weight = self.weight.reshape(1).expand(self.width).contiguous()
        if self.unit_offset:
            self.weight = (self.weight + 1.0).contiguous()
        if self.scale != 1.0:
            self.weight = (self.weight * self.scale).contiguous()

    def deferred(self):
        if self.opts.dtype != torch.bfloat16 or self.weight is None:
            return None
        return self.weight, self.width, self.eps

    def forward(self, residual, delta, out=None, rows=None, n_rows=None):
        if out is None:
            n = (rows.numel() if rows is not None else residual.shape[0]) if n_rows is None else n_rows
            out = torch.empty((max(n, 0) if rows is not None else residual.shape[0], self.width),
                              dtype=self.opts.dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows, n_rows=n_rows)
