"""Grouped-query attention over the paged cache in its wider forms: keys and values of sizes of their own,
several score maps per head, query and key norm, values that are the keys as projected, a sink, a window.

H query heads share G key/value heads (head h reads group h // (H/G)).  A head has M score maps; its query
has M vectors of `dim`, a group has M key vectors of `dim` and ONE value vector of `vdim`; the rows of W_q
and W_k are laid out head by head as [map 0, map 1, ..].  Per map m:

    a_m = softmax_s((q_m . k_m,s) * scale) v_s       over the keys s with 0 <= p - s < window

With `sink`, exp(sink_h) is one more term of every softmax's denominator (no key, no value, not scaled).
Options, each a constructor argument:

    qk_norm          q and k vectors are divided by their root mean square and multiplied by a weight of size
                     `dim` (one for all query heads, one for all key heads), before the rotation
    values_are_keys  there is no W_v: the values are the key vectors as projected, before norm and rotation
    difference d     M = 2: o = a_0 - lambda a_1 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + d from four
                     learned vectors of size `dim`; o is then divided by its root mean square over `vdim` (no
                     weight) and multiplied by 1 - d.  (Ye et al., "Differential Transformer".)

    qk_norm_weight   off: the query/key norm has no weight (and no tensors)
    value_norm       every value vector is divided by its root mean square over `vdim` (no weight) before it is cached
    head_mix         a matrix T [H, H] (tensor `<prefix>.<head_mix>`) mixes the softmax weights of all heads before they
                     meet the values: w'_h = sum_g T[h, g] w_g, and head h applies w'_h to the values of its own
                     key/value head (Shazeer et al., "Talking-Heads Attention", mix after the softmax like this).
                     One map, no sink.  The cache keeps a token's value heads side by side in one row, head g's
                     attention over that whole row is computed once, and o_h = sum_g T[h, g] A[g, group of h]; the
                     rows of W_q are reordered at load so that neighbouring query vectors read different key heads.
    gate             the concatenated heads are multiplied by sigmoid(W_g h) (tensor `<prefix>.<gate>`) before W_o
    head_gate        every head's output is multiplied by sigmoid(W_g h)_h, ONE number per head and token (tensor
                     `<prefix>.<head_gate>` [H, width]), before W_o; its rows ride in the projections' product

The rotation turns the first n_rot dims of every query and key vector (each map by itself).  In bfloat16 with key
and value sizes in steps of 16, prompts and decode steps run on the tensor-core kernels of csrc/attention_mma.cu
(several maps leave their outputs in float32, which one more kernel combines); everything else runs
csrc/attention_maps.cu (32-bit arithmetic).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, KVSpec, Mixer, PositionEncoding
from .linear import Linear


class MapsAttention(Mixer):
    def __init__(self, opts: BuildOptions, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int | None,
                 position: PositionEncoding | None, prefix: str, scale: float, eps: float, window: int | None = None,
                 n_maps: int = 1, bias: bool = False, qk_norm: bool = False, values_are_keys: bool = False,
                 sink: bool = False, difference: float | None = None, names=("q", "k", "v", "o"),
                 weight_suffix: str = "", bias_suffix: str = ".b", out_dtype=None, qk_norm_weight: bool = True,
                 value_norm: bool = False, head_mix: str | None = None, gate: str | None = None,
                 head_gate: str | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{prefix}: {n_heads} heads cannot share {n_kv_heads} key/value heads")
        self.opts, self.prefix = opts, prefix
        self.width, self.H, self.G, self.M, self.Dk = int(width), int(n_heads), int(n_kv_heads), int(n_maps), int(dim)
        self.values_are_keys = bool(values_are_keys)
        if self.values_are_keys:
            if self.M != 1 or (vdim is not None and int(vdim) != self.Dk):
                raise ValueError(f"{prefix}: values that are the keys need one map and a value size equal to the keys'")
            vdim = self.Dk
        self.Dv = int(vdim if vdim is not None else dim)
        if difference is not None and self.M != 2:
            raise ValueError(f"{prefix}: the difference of maps needs exactly two maps")
        big = ops.ATTENTION_MAPS_MAX_DIM
        if not (0 < self.Dk <= big and 0 < self.Dv <= big):
            raise ValueError(f"{prefix}: head sizes {self.Dk} and {self.Dv} are outside 1..{big}")
        self.qk_norm_weight, self.value_norm, self.head_mix, self.gate = bool(qk_norm_weight), bool(value_norm), head_mix, gate
        self.head_gate = head_gate
        if head_gate is not None and (gate is not None or head_mix is not None):
            raise ValueError(f"{prefix}: a gate per head stands alone (no gate per value, no mixed heads)")
        if gate is not None and head_mix is None:
            raise ValueError(f"{prefix}: the output gate is applied by the kernel that mixes the heads (head_mix)")
        if head_mix is not None:
            if self.M != 1 or sink or self.values_are_keys:
                raise ValueError(f"{prefix}: mixed heads need one map, no sink and values of their own")
            if self.G * self.Dv > ops.talk_max_row():
                raise ValueError(f"{prefix}: {self.G} value heads of {self.Dv} are more than {ops.talk_max_row()} numbers per token")
        self.window = int(window) if window else None
        self.scale, self.eps = float(scale), float(eps)
        self.position, self.qk_norm, self.has_sink = position, bool(qk_norm), bool(sink)
        self.difference = None if difference is None else float(difference)
        q, k, v, o = names
        self.names = names
        n_q, n_k = self.H * self.M * self.Dk, self.G * self.M * self.Dk
        sources = [(f"{prefix}.{q}", n_q), (f"{prefix}.{k}", n_k)]
        if not self.values_are_keys:
            sources.append((f"{prefix}.{v}", self.G * self.Dv))
        self.offsets = (0, n_q, n_q if self.values_are_keys else n_q + n_k)
        self.gate_offset = None
        if gate is not None:
            self.gate_offset = sum(r for _, r in sources)
            sources.append((f"{prefix}.{gate}", self.H * self.Dv))
        pad = 0
        if head_gate is not None:
            sources.append((f"{prefix}.{head_gate}", self.H))
            # the tcgen05 prefill kernel reads the product's rows as [token, head, dim]: the H gate rows are padded
            # (with zero rows, at load) so that a token's row stays a whole number of heads
            if self.Dk == self.Dv and self.Dk in (64, 128) and self.M == 1:
                pad = self.Dk
        self.qkv = Linear(opts, width, sources, bias=bias, weight_suffix=weight_suffix, bias_suffix=bias_suffix,
                          pad_rows_to=pad)
        if head_gate is not None:
            self.gate_offset = sum(r for _, r in self.qkv.sources[:-1])
        self.out = Linear(opts, self.H * self.Dv, [(f"{prefix}.{o}", width)], weight_suffix=weight_suffix,
                          out_dtype=out_dtype)
        self.q_weight = self.k_weight = self.sink = self.talk = None
        self.coef = 0.0

    def own_param_specs(self):
        p, (q, k, _, _) = self.prefix, self.names
        specs = []
        if self.difference is not None:
            specs += [ParamSpec(f"{p}.{n}", (self.Dk,), "vector", "normal") for n in ("lq1", "lk1", "lq2", "lk2")]
        if self.qk_norm and self.qk_norm_weight:
            specs += [ParamSpec(f"{p}.{q}.norm", (self.Dk,), "vector", "one_plus_normal"),
                      ParamSpec(f"{p}.{k}.norm", (self.Dk,), "vector", "one_plus_normal")]
        if self.head_mix is not None:
            specs.append(ParamSpec(f"{p}.{self.head_mix}", (self.H, self.H), "vector", "normal"))
        if self.has_sink:
            specs.append(ParamSpec(f"{p}.sink", (self.H,), "vector", "normal"))
        return specs

    def load_own(self, fetch):
        got = {s.name[len(self.prefix) + 1:]: fetch(s) for s in self.own_param_specs()}
        if self.difference is not None:
            d = {n: got[n].double().cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
            lam = (math.exp(float((d["lq1"] * d["lk1"]).sum())) - math.exp(float((d["lq2"] * d["lk2"]).sum()))
                   + self.difference)
            self.coef = -lam
        if self.qk_norm and self.qk_norm_weight:
            self.q_weight, self.k_weight = got[f"{self.names[0]}.norm"], got[f"{self.names[1]}.norm"]
        elif self.qk_norm:
            self.q_weight = self.k_weight = torch.ones(self.Dk, dtype=torch.float32, device=self.opts.device)
        if self.head_mix is not None:
            self.talk = got[self.head_mix].contiguous()
        if self.has_sink:
            self.sink = got["sink"]

    def load(self, fetch):
        super().load(fetch)
        if self.head_mix is not None:
            # query vector x = j * G + c is head c * (H/G) + j: neighbours read different key heads
            n_q, per = self.H * self.Dk, self.H // self.G
            w = self.qkv.weight
            w[:n_q] = w[:n_q].reshape(self.G, per, self.Dk, -1).transpose(0, 1).reshape(n_q, -1).clone()
            if self.qkv.bias is not None:
                b = self.qkv.bias
                b[:n_q] = b[:n_q].reshape(self.G, per, self.Dk).transpose(0, 1).reshape(n_q).clone()

    def cache_spec(self):
        if self.head_mix is not None:       # a token's value heads side by side in one row
            return KVSpec(self.G, self.Dk, self.window, value_heads=1, value_dim=self.G * self.Dv)
        return KVSpec(self.G * self.M, self.Dk, self.window, value_heads=self.G, value_dim=self.Dv)

    def _on_tensor_cores(self, buf) -> bool:
        return ops.attention_maps_mma_supports(self.H, self.G, self.M, self.Dk, self.Dv, buf.shape[-1], buf.dtype)

    adds_to_residual = True

    def forward(self, h, ctx, cache, write_cache: bool = True, then=None):
        T = ctx.n_tokens
        # many rows in bfloat16: the library product has no bias in it, and the kernel that prepares q and k
        # touches every projected value anyway; few rows and the 32-bit path add it in the product
        later = self.qkv.bias is not None and h.dtype == torch.bfloat16 and T > ops.GEMV_NARROW_MAX_ROWS
        buf = self.qkv.forward(h, n_rows=T, with_bias=not later)
        rot = self.position.rotation() if self.position is not None else None
        ops.attention_prepare(buf, self.offsets, self.H, self.G, self.M, self.Dk, self.Dv, cache, ctx,
                              q_weight=self.q_weight, k_weight=self.k_weight, eps=self.eps, rot=rot,
                              write_cache=write_cache, bias=self.qkv.bias if later else None,
                              v_norm=self.value_norm, v_side_by_side=self.head_mix is not None)
        att = torch.empty((buf.shape[0], self.H * self.Dv), dtype=buf.dtype, device=buf.device)
        if self.head_mix is not None:
            gate_rows = buf.reshape(-1)[self.gate_offset:] if self.gate_offset is not None else None
            ops.attention_talk(buf, buf.shape[-1], att, cache, ctx, self.H, self.G, self.Dk, self.Dv, self.scale,
                               self.talk, gate_rows=gate_rows, gate_stride=buf.shape[-1], window=self.window or 0)
            return self.out.forward(att, n_rows=T, start_early=False, then=then)

        unit = self.difference is not None
        attend = ops.attention_maps_mma if self._on_tensor_cores(buf) else ops.attention_maps
        attend(buf, buf.shape[-1], att, cache, ctx, self.H, self.G, self.M, self.Dk, self.Dv, self.scale,
               self.window or 0, self.sink, coef=self.coef, unit_norm=unit, eps=self.eps,
               out_scale=(1.0 - self.difference) if unit else 1.0)
        if self.head_gate is not None:
            ops.head_gate(att, buf.reshape(-1)[self.gate_offset:], buf.shape[-1], T, self.H, self.Dv)
        # after a kernel that fills the processors' shared memory the product starts when that kernel has ended
        return self.out.forward(att, n_rows=T, start_early=False, then=then)
