"""Recurrent mixers whose state decays by amounts that depend on the token.  Both keep one matrix S [D, V] per
(sequence, head) in float32, zero at a sequence's start, carried from step to step; a prompt may be cut anywhere and
a decode step is a step of one token.

`GatedLinearAttention`: a decay per key channel (Yang et al., "Gated Linear Attention Transformers with
Hardware-Efficient Training"):

    q = W_q h * D^(-1/2), k = W_k h (H x D), v = W_v h (H x V)
    a = sigmoid(W_a2 (W_a1 h) + b)^(1/tau)                      H x D numbers in (0, 1) per token
    S <- diag(a) S + k v^T;   o = S^T q
    out = W_o (rmsnorm_V(o) * w * silu(W_g h))                  one weight w [V] for all heads

`GatedDeltaRule`: one decay per head and a write that first takes back what the key already reads (Yang et al.,
"Gated Delta Networks: Improving Mamba2 with Delta Rule"):

    q, k = W h (G x D), v = W_v h (H x V): each passes a short causal convolution per channel over time and SiLU
    q, k -> unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times D^(-1/2); head h reads q/k head h // (H/G)
    beta = sigmoid(W_b h);   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))          per head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out = W_o (rmsnorm_V(o) * w * silu(W_g h))

The convolution's last taps - 1 inputs are a second state of the sequence.  The projections are one product with a
float32 result; everything after it up to the output projection is 32-bit arithmetic (csrc/gated_recurrence.cu).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Mixer, StateSpec
from .linear import Linear


class GatedLinearAttention(Mixer):
    def __init__(self, opts: BuildOptions, width: int, n_heads: int, dim: int, vdim: int, rank: int, tau: float, eps: float,
                 prefix: str, names=("q", "k", "v", "g", "o", "norm", "a1", "a2"), weight_suffix: str = "",
                 bias_suffix: str = ".b", out_dtype=None):
        self.opts = opts
        self.width, self.H, self.D, self.V, self.rank = int(width), int(n_heads), int(dim), int(vdim), int(rank)
        self.tau, self.eps, self.prefix, self.names = float(tau), float(eps), prefix, names
        self.bias_suffix = bias_suffix
        if not 0 < self.D <= ops.RECURRENCE_MAX_DIM:
            raise ValueError(f"{prefix}: {self.D} dims per head are outside 1..{ops.RECURRENCE_MAX_DIM}")
        if not self.tau > 0:
            raise ValueError(f"{prefix}: tau must be positive, got {tau}")
        q, k, v, g, o, _, a1, _ = names
        H, D, V = self.H, self.D, self.V
        rows = [(q, H * D), (k, H * D), (v, H * V), (g, H * V), (a1, self.rank)]
        self.offsets, at = [], 0
        for _, r in rows:
            self.offsets.append(at)
            at += r
        # what enters the recurrence is 32-bit: the projections leave the product in float32
        self.proj = Linear(opts, width, [(f"{prefix}.{n}", r) for n, r in rows], out_dtype=torch.float32,
                           weight_suffix=weight_suffix)
        self.out = Linear(opts, H * V, [(f"{prefix}.{o}", width)], weight_suffix=weight_suffix, out_dtype=out_dtype)
        self.norm_weight = self.w_a2 = self.b_a2 = None

    def own_param_specs(self):
        p, n = self.prefix, self.names
        return [ParamSpec(f"{p}.{n[5]}", (self.V,), "vector", "one_plus_normal"),
                ParamSpec(f"{p}.{n[7]}", (self.H * self.D, self.rank), "vector", "normal"),
                ParamSpec(f"{p}.{n[7]}{self.bias_suffix}", (self.H * self.D,), "vector", "normal")]

    def load_own(self, fetch):
        self.norm_weight, w_a2, self.b_a2 = (fetch(s) for s in self.own_param_specs())
        self.w_a2 = w_a2.t().contiguous()          # [rank, H * D]: what the kernel reads

    def cache_spec(self):
        return StateSpec((self.H, self.D, self.V), torch.float32)

    def forward(self, h, ctx, cache, write_cache: bool = True):
        T, H, D, V = ctx.n_tokens, self.H, self.D, self.V
        proj = self.proj.forward(h, n_rows=T)
        oq, ok, ov, og, oa = self.offsets
        decay = torch.empty((proj.shape[0], H * D), dtype=torch.float32, device=proj.device)
        ops.gla_decay(proj[:, oa:oa + self.rank], self.w_a2, self.b_a2, self.tau, decay, T)
        o = torch.empty((proj.shape[0], H * V), dtype=torch.float32, device=proj.device)
        ops.gated_recurrence("channel", proj[:, oq:oq + H * D], proj[:, ok:ok + H * D], proj[:, ov:ov + H * V],
                             cache.state, o, ctx, H, H, D, V, qscale=float(D) ** -0.5, decay=decay,
                             write_state=write_cache)
        mixed = torch.empty((proj.shape[0], H * V), dtype=self.opts.dtype, device=proj.device)
        ops.head_norm_gate(o, self.norm_weight, proj[:, og:og + H * V], "silu", self.eps, mixed, ctx, H, V)
        return self.out.forward(mixed, n_rows=T)


class GatedDeltaRule(Mixer):
    UNIT_EPS = 1e-6       # inside the root of the unit vectors' lengths

    def __init__(self, opts: BuildOptions, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, taps: int,
                 eps: float, prefix: str, names=("q", "k", "v", "b", "a", "g", "o", "norm", "A_log", "dt_bias"),
                 conv_suffix: str = ".conv", weight_suffix: str = "", out_dtype=None):
        self.opts = opts
        self.width, self.H, self.G, self.D, self.V = int(width), int(n_heads), int(n_kv_heads), int(dim), int(vdim)
        self.taps, self.eps, self.prefix, self.names, self.conv_suffix = int(taps), float(eps), prefix, names, conv_suffix
        if self.H % self.G:
            raise ValueError(f"{prefix}: {self.H} heads cannot share {self.G} query/key heads")
        if not 0 < self.D <= ops.RECURRENCE_MAX_DIM:
            raise ValueError(f"{prefix}: {self.D} dims per head are outside 1..{ops.RECURRENCE_MAX_DIM}")
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"{prefix}: a convolution over {self.taps} tokens is outside 1..{ops.CONV_MAX_TAPS}")
        q, k, v, b, a, g, o = names[:7]
        H, G, D, V = self.H, self.G, self.D, self.V
        rows = [(q, G * D), (k, G * D), (v, H * V), (b, H), (a, H), (g, H * V)]
        self.offsets, at = [], 0
        for _, r in rows:
            self.offsets.append(at)
            at += r
        self.channels = 2 * G * D + H * V
        self.proj = Linear(opts, width, [(f"{prefix}.{n}", r) for n, r in rows], out_dtype=torch.float32,
                           weight_suffix=weight_suffix)
        self.out = Linear(opts, H * V, [(f"{prefix}.{o}", width)], weight_suffix=weight_suffix, out_dtype=out_dtype)
        self.norm_weight = self.A_log = self.dt_bias = self.conv = None

    def own_param_specs(self):
        p, n, c = self.prefix, self.names, self.conv_suffix
        return [ParamSpec(f"{p}.{n[7]}", (self.V,), "vector", "one_plus_normal"),
                ParamSpec(f"{p}.{n[8]}", (self.H,), "vector", "normal"),
                ParamSpec(f"{p}.{n[9]}", (self.H,), "vector", "normal"),
                ParamSpec(f"{p}.{n[0]}{c}", (self.G * self.D, self.taps), "vector", "normal"),
                ParamSpec(f"{p}.{n[1]}{c}", (self.G * self.D, self.taps), "vector", "normal"),
                ParamSpec(f"{p}.{n[2]}{c}", (self.H * self.V, self.taps), "vector", "normal")]

    def load_own(self, fetch):
        specs = self.own_param_specs()
        self.norm_weight, self.A_log, self.dt_bias = (fetch(s) for s in specs[:3])
        self.conv = torch.cat([fetch(s) for s in specs[3:]], dim=0).contiguous()       # [channels, taps], q | k | v

    def cache_specs(self) -> list:
        """The matrix per head, and the convolution's last inputs."""
        return [StateSpec((self.H, self.D, self.V), torch.float32),
                StateSpec((max(self.taps - 1, 1), self.channels), torch.float32)]

    def cache_spec(self):
        raise ValueError(f"{self.prefix}: the mixer keeps two states; the block asks `cache_specs()`")

    def forward(self, h, ctx, cache, write_cache: bool = True):
        T, H, G, D, V = ctx.n_tokens, self.H, self.G, self.D, self.V
        memory, held = cache
        proj = self.proj.forward(h, n_rows=T)
        oq, ok, ov, ob, oa, og = self.offsets
        dev, rows = proj.device, proj.shape[0]
        qkv = torch.empty((rows, self.channels), dtype=torch.float32, device=dev)
        beta = torch.empty((rows, H), dtype=torch.float32, device=dev)
        decay = torch.empty((rows, H), dtype=torch.float32, device=dev)
        ops.gdr_prepare(proj, self.conv, held.state, self.A_log, self.dt_bias, ob, oa, float(D) ** -0.5, self.UNIT_EPS,
                        qkv, beta, decay, ctx, H, G, D, V, write_state=write_cache)
        o = torch.empty((rows, H * V), dtype=torch.float32, device=dev)
        ops.gated_recurrence("delta", qkv[:, :G * D], qkv[:, G * D:2 * G * D], qkv[:, 2 * G * D:], memory.state, o, ctx,
                             H, G, D, V, decay=decay, beta=beta, write_state=write_cache)
        mixed = torch.empty((rows, H * V), dtype=self.opts.dtype, device=dev)
        ops.head_norm_gate(o, self.norm_weight, proj[:, og:og + H * V], "silu", self.eps, mixed, ctx, H, V)
        return self.out.forward(mixed, n_rows=T)
