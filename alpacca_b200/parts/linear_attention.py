"""Linear attention with a fixed decay per head ("lightning attention") as a mixer with a state of fixed size
per sequence.

Per head, q = silu(W_q h), k = silu(W_k h) (D dims each), v = silu(W_v h) (V dims), a decay 0 < a <= 1 that is
a constant of the head, and S = 0 before the first token:

    S' = a S + k v^T;   o = S'^T q          (no other scale)

The heads of a token are concatenated, divided by their common root mean square, multiplied by a weight and
by sigmoid(W_g h), and projected by W_o.  (Qin et al., "Lightning Attention-2: A Free Lunch for Handling
Unlimited Sequence Lengths in Large Language Models", describe the recurrence and its block form.)

Options, each a constructor argument (the retention of Sun et al., "Retentive Network: A Successor to Transformer
for Large Language Models", is this recurrence with rotated q and k, no activation, a norm per head and a SiLU gate):

    activation     "silu" (above) or None: q, k, v enter as projected
    position       a rotation of the first n_rot dims of every q and k vector by the token's position
    key_scale      k is multiplied by this constant after the rotation
    head_norm      the root mean square is taken per head (V values) instead of over all heads
    norm_weight    off: the norm has no weight (and no tensor)
    gate           "sigmoid" or "silu" of W_g h

The four projections are one product with a float32 result; the activations, the decay, the state and the
normalisation are 32-bit arithmetic in both precisions (csrc/linear_attention.cu).  The state lives in the
cache's state group, one [D, V] matrix per (slot, head), and is carried from step to step: a prompt may be cut
anywhere, and a decode step is a step of one token.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Mixer, StateSpec
from .linear import Linear


class DecayLinearAttention(Mixer):
    def __init__(self, opts: BuildOptions, width: int, n_heads: int, dim: int, vdim: int, decay, eps: float,
                 prefix: str, names=("q", "k", "v", "g", "o", "norm"), weight_suffix: str = "", out_dtype=None,
                 activation: str | None = "silu", position=None, key_scale: float = 1.0, head_norm: bool = False,
                 norm_weight: bool = True, gate: str = "sigmoid"):
        self.opts = opts
        self.width, self.H, self.D, self.V = int(width), int(n_heads), int(dim), int(vdim)
        self.eps, self.prefix, self.names = float(eps), prefix, names
        decay = [float(a) for a in decay]
        if len(decay) != self.H or not all(0.0 < a <= 1.0 for a in decay):
            raise ValueError(f"{prefix}: {self.H} decays in (0, 1] are needed, got {decay}")
        if not 0 < self.D <= ops.linear_attention_max_dim():
            raise ValueError(f"{prefix}: {self.D} dims per head are outside 1..{ops.linear_attention_max_dim()}")
        if activation not in ("silu", None) or gate not in ("sigmoid", "silu"):
            raise ValueError(f"{prefix}: activation {activation!r} (silu or None) or gate {gate!r} (sigmoid, silu) unknown")
        if not norm_weight and not head_norm:
            raise ValueError(f"{prefix}: the norm over all heads has a weight")
        self.activation, self.position, self.key_scale = activation, position, float(key_scale)
        self.head_norm, self.has_norm_weight, self.gate = bool(head_norm), bool(norm_weight), gate
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(opts.device)
        q, k, v, g, o, _ = names
        H, D, V = self.H, self.D, self.V
        rows = [(q, H * D), (k, H * D), (v, H * V), (g, H * V)]
        self.offsets, at = [], 0
        for _, r in rows:
            self.offsets.append(at)
            at += r
        # what enters the recurrence is 32-bit: the projections leave the product in float32
        self.proj = Linear(opts, width, [(f"{prefix}.{n}", r) for n, r in rows], out_dtype=torch.float32,
                           weight_suffix=weight_suffix)
        self.out = Linear(opts, H * V, [(f"{prefix}.{o}", width)], weight_suffix=weight_suffix, out_dtype=out_dtype)
        self.norm_weight = None

    def children(self):
        return [self.proj, self.out]          # a rotation table is shared between layers and has no tensors

    def own_param_specs(self):
        if not self.has_norm_weight:
            return []
        return [ParamSpec(f"{self.prefix}.{self.names[5]}", (self.H * self.V,), "vector", "one_plus_normal")]

    def load_own(self, fetch):
        if self.has_norm_weight:
            self.norm_weight = fetch(self.own_param_specs()[0])

    def cache_spec(self):
        return StateSpec((self.H, self.D, self.V), torch.float32)

    adds_to_residual = True

    def forward(self, h, ctx, cache, write_cache: bool = True, then=None):
        T = ctx.n_tokens
        proj = self.proj.forward(h, n_rows=T)
        mixed = torch.empty((proj.shape[0], self.H * self.V), dtype=self.opts.dtype, device=proj.device)
        ops.linear_attention_step(proj, self.offsets, self.decay, cache.state, ctx, self.H, self.D, self.V,
                                  self.norm_weight, self.eps, mixed, write_state=write_cache,
                                  activation=self.activation == "silu",
                                  rot=self.position.rotation() if self.position is not None else None,
                                  k_scale=self.key_scale, head_norm=self.head_norm, gate=self.gate)
        return self.out.forward(mixed, n_rows=T, then=then)
