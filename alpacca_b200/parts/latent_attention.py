"""Causal attention whose keys and values are kept as one low-rank latent per token.

    c_q = RMSnorm(W_dq h) * w_q;  q = W_uq c_q, per head [D unrotated | R rotated] dims
    W_dkv h = [C | R] rows:  c = RMSnorm(first C) * w_c;  r = the last R, rotated by position, one for all heads
    per head: k = W_uk c (D dims), v = W_uv c (V dims); score = (q_un . k + q_rot . r) * scale, keys up to the
    token's own position; softmax whose denominator also holds exp(sink_h); output W_o on the heads' values

Only [c | r] is cached: one row of C + R numbers per token, in pages of the cache's key/value kind without a
value tensor.  The up-projection of the keys is folded into the query (q' = W_uk_h^T q_un, C dims), so a
score is q' . c + q_rot . r on the cached row itself, and the values' up-projection is applied to the
attention's weighted sum of c: nothing is expanded per cached token, in prompts and decode steps alike.
(The latent form is DeepSeek-V2's multi-head latent attention; the sink is a learned logit per head.)

Options, each a constructor argument:

    sink          off: an ordinary softmax (and no tensor)
    window        a token sees itself and the window - 1 tokens before it
    keep_window   what the cache keeps, where it must be more than this layer reads: another layer may read this
                  layer's latent rows with a window of its own (the cache entry is then sized for the largest)
    head_gate     every head's output is multiplied by sigmoid(W_g h)_h, one number per head and token (tensor
                  `<prefix>.<head_gate>` [H, width]); its rows ride in the down-projections' product
    own_kv        off: the layer has no W_dkv; it reads the latent rows that another layer of the same kv_rank, rot_dim
                  and rotation has cached (the schedule's run names that layer's run), with its own W_uk, W_uv, queries,
                  window and gate

Norms, rotation, scores, softmax and the weighted sum are 32-bit arithmetic (csrc/latent_attention.cu).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, KVSpec, Mixer, PositionEncoding
from .linear import Linear


class LatentAttention(Mixer):
    def __init__(self, opts: BuildOptions, width: int, n_heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, position: PositionEncoding | None, prefix: str,
                 sink: bool = True, names=("dq", "uq", "dkv", "uk", "uv", "o", "sink"), norm_suffix: str = ".norm",
                 weight_suffix: str = "", out_dtype=None, window: int | None = None, keep_window: int | None = None,
                 head_gate: str | None = None, own_kv: bool = True):
        self.opts = opts
        self.window = int(window) if window else None
        self.keep_window = (int(keep_window) if keep_window else None) if keep_window != "all" else None
        if self.window is None or keep_window == "all":
            self.keep_window = None            # a layer that reads everything keeps everything
        elif self.keep_window is None:
            self.keep_window = self.window
        elif self.keep_window < self.window:
            raise ValueError(f"{prefix}: the cache keeps {self.keep_window} tokens, the window reads {self.window}")
        self.head_gate, self.own_kv = head_gate, bool(own_kv)
        self.width, self.H, self.D, self.R, self.V = int(width), int(n_heads), int(dim), int(rot_dim), int(vdim)
        self.Q, self.C = int(q_rank), int(kv_rank)
        self.scale, self.eps, self.position, self.prefix = float(scale), float(eps), position, prefix
        self.has_sink, self.names, self.norm_suffix, self.weight_suffix = bool(sink), names, norm_suffix, weight_suffix
        dq, uq, dkv, uk, uv, o, _ = names
        H, D, R, V, Q, C = self.H, self.D, self.R, self.V, self.Q, self.C
        # both down-projections read the same input: one product, float32 result (it feeds two norms)
        sources = [(f"{prefix}.{dq}", Q)] + ([(f"{prefix}.{dkv}", C + R)] if self.own_kv else [])
        self.gate_offset = sum(r for _, r in sources)
        if head_gate is not None:
            sources.append((f"{prefix}.{head_gate}", H))
        self.down = Linear(opts, width, sources, out_dtype=torch.float32, weight_suffix=weight_suffix)
        self.up_q = Linear(opts, Q, [(f"{prefix}.{uq}", H * (D + R))], weight_suffix=weight_suffix)
        self.out = Linear(opts, H * V, [(f"{prefix}.{o}", width)], weight_suffix=weight_suffix, out_dtype=out_dtype)
        self.q_norm = self.c_norm = self.sink = None
        self.w_uk_t = self.w_uv = None        # [H, C, D] (transposed per head) and [H, V, C]: what the kernel reads
        self.w_uk = self.w_uv_t = None        # [H, D, C] and [H, C, V]: the right-hand sides of library products

    def own_param_specs(self):
        dq, _, dkv, uk, uv, _, sink = self.names
        p, s = self.prefix, self.weight_suffix
        specs = [ParamSpec(f"{p}.{dq}{self.norm_suffix}", (self.Q,), "vector", "one_plus_normal"),
                 ParamSpec(f"{p}.{dkv}{self.norm_suffix}", (self.C,), "vector", "one_plus_normal", absent=not self.own_kv),
                 ParamSpec(f"{p}.{uk}{s}", (self.H * self.D, self.C), "matrix", "normal"),
                 ParamSpec(f"{p}.{uv}{s}", (self.H * self.V, self.C), "matrix", "normal")]
        if self.has_sink:
            specs.append(ParamSpec(f"{p}.{sink}", (self.H,), "vector", "normal"))
        return specs

    def load_own(self, fetch):
        specs = self.own_param_specs()
        self.q_norm, self.c_norm = fetch(specs[0]), (fetch(specs[1]) if self.own_kv else None)
        uk, uv = fetch(specs[2]), fetch(specs[3])
        self.w_uk = uk.view(self.H, self.D, self.C).contiguous()
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous()
        self.w_uv = uv.view(self.H, self.V, self.C).contiguous()
        self.w_uv_t = self.w_uv.transpose(1, 2).contiguous()
        self.sink = fetch(specs[4]) if self.has_sink else None

    def cache_spec(self):
        return KVSpec(1, self.C + self.R, self.keep_window, values=False)

    def forward(self, h, ctx, cache, write_cache: bool = True):
        T = ctx.n_tokens
        H, D, R, V, Q, C = self.H, self.D, self.R, self.V, self.Q, self.C
        dev = h.device
        down = self.down.forward(h, n_rows=T)
        rot = self.position.rotation() if self.position is not None else None
        cq = torch.empty((down.shape[0], Q), dtype=self.opts.dtype, device=dev)
        if write_cache and not self.own_kv:
            raise ValueError(f"{self.prefix}: a layer without W_dkv writes no cache; its run reads another run's")
        ops.latent_prep(down, Q, C, R, self.q_norm, self.c_norm, self.eps, rot, ctx, cache, cq,
                        write_cache=write_cache and self.own_kv)
        q = self.up_q.forward(cq, n_rows=T)
        gate = down.reshape(-1)[self.gate_offset:] if self.head_gate is not None else None
        if ops.latent_attention_mma_supports(H, C, R, self.opts.dtype):
            return self._forward_tensor_cores(q, rot, ctx, cache, gate, down.shape[-1])
        q_lat = torch.empty((q.shape[0], H * (C + R)), dtype=torch.float32, device=dev)
        ops.heads_matmul(q, D + R, self.w_uk_t, q_lat, C + R, T, tail=R, rot=rot, ctx=ctx)
        o_lat = torch.empty((q.shape[0], H * C), dtype=torch.float32, device=dev)
        ops.latent_attention(q_lat, o_lat, cache, ctx, H, C, R, self.scale, self.sink, window=self.window or 0)
        values = torch.empty((q.shape[0], H * V), dtype=self.opts.dtype, device=dev)
        ops.heads_matmul(o_lat, C, self.w_uv, values, V, T, ctx=ctx)
        if gate is not None:
            ops.head_gate(values, gate, down.shape[-1], T, H, V)
        return self.out.forward(values, n_rows=T)

    def _forward_tensor_cores(self, q, rot, ctx, cache, gate=None, gate_stride=0):
        """bfloat16, rows of up to 256 dims: the folded query and the heads' outputs are bfloat16, the attention
        runs on the tensor-core kernels; the per-head products are library products from 17 rows on."""
        T = ctx.n_tokens
        H, D, R, V, C = self.H, self.D, self.R, self.V, self.C
        Dk = C + R
        rows, dev = q.shape[0], q.device
        many = T >= ops.LIBRARY_HEADS_MIN_ROWS
        q_lat = torch.empty((rows, H * Dk), dtype=torch.bfloat16, device=dev)
        if many:
            ops.heads_mm_library(q, D + R, D, self.w_uk, q_lat, Dk, T)
            ops.heads_matmul(q, D + R, None, q_lat, Dk, T, tail=R, rot=rot, ctx=ctx, tail_at=C)
        else:
            ops.heads_matmul(q, D + R, self.w_uk_t, q_lat, Dk, T, tail=R, rot=rot, ctx=ctx)
        o_lat = torch.empty((rows, H * Dk), dtype=torch.bfloat16, device=dev)
        ops.latent_attention_mma(q_lat, o_lat, cache, ctx, H, C, R, self.scale, self.sink, window=self.window or 0)
        values = torch.empty((rows, H * V), dtype=torch.bfloat16, device=dev)
        if many:
            ops.heads_mm_library(o_lat, Dk, C, self.w_uv_t, values, V, T)
        else:
            ops.heads_matmul(o_lat, Dk, self.w_uv, values, V, T, ctx=ctx)
        if gate is not None:
            ops.head_gate(values, gate, gate_stride, T, H, V)
        return self.out.forward(values, n_rows=T)
