"""Token embedding (row gather, no scaling: alpacca/model.py:482; options: a constant factor, and a hashed table
of (previous token, token) pairs whose row is added) and the
vocabulary head (logits = W . norm(x), alpacca/model.py:518; tied: the head is
the embedding table itself, :320-322).  Logits are float32 in both precisions.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Part, StateSpec
from .linear import Linear


class PairTable(Part):
    """A table of `buckets` + 1 rows for pairs of neighbouring tokens: a token after `prev` reads row
    (prev * mul_prev + token * mul_cur) mod buckets, a sequence's first token the last row."""

    def __init__(self, opts: BuildOptions, buckets: int, width: int, mul_prev: int, mul_cur: int, name: str):
        self.opts, self.buckets, self.width, self.name = opts, int(buckets), int(width), name
        self.mul_prev, self.mul_cur = int(mul_prev), int(mul_cur)
        if self.buckets <= 0 or not (0 <= self.mul_prev < 2 ** 31 and 0 <= self.mul_cur < 2 ** 31):
            raise ValueError(f"{name}: {buckets} buckets and multipliers {mul_prev}, {mul_cur} cannot index a table")
        self.weight = None

    def own_param_specs(self):
        return [ParamSpec(self.name, (self.buckets + 1, self.width), "matrix", "normal")]

    def load_own(self, fetch):
        self.weight = fetch(self.own_param_specs()[0])


class TokenEmbedding(Part):
    def __init__(self, opts: BuildOptions, vocab: int, width: int, name: str, weight_suffix: str = ".weight",
                 norm=None, scale: float = 1.0, pairs: "PairTable | None" = None):
        """`norm`: a norm that the embedded rows pass before they become the stream (32-bit).  `scale`: a factor on
        the embedded row.  `pairs`: a `PairTable` whose row for (previous token, token) is added (not scaled); the
        sequence's last token is then part of what it keeps from step to step (`cache_spec`)."""
        self.opts, self.vocab, self.width, self.name = opts, int(vocab), int(width), name
        self.weight_suffix = weight_suffix
        self.weight = None
        self.norm = norm
        self.scale, self.pairs = float(scale), pairs
        if norm is not None and (pairs is not None or self.scale != 1.0):
            raise ValueError(f"{name}: a normed embedding has no factor and no pair table")

    def cache_spec(self):
        """What the embedding keeps per sequence: its last token, for the pair of the next step's first token."""
        return StateSpec((1,), torch.int32) if self.pairs is not None else None

    def own_param_specs(self):
        return [ParamSpec(f"{self.name}{self.weight_suffix}", (self.vocab, self.width), "matrix", "normal")]

    def load_own(self, fetch):
        self.weight = fetch(self.own_param_specs()[0])

    def forward(self, tokens: torch.Tensor, n_rows: int, ctx=None, cache=None) -> torch.Tensor:
        out = torch.empty((n_rows, self.width), dtype=torch.float32, device=tokens.device)
        if self.pairs is not None or self.scale != 1.0:
            if ctx is None or (self.pairs is not None and cache is None):
                raise ValueError(f"{self.name}: the embedding needs the step's context (and the sequences' last tokens)")
            p = self.pairs
            if p is None:
                return ops.embed_pairs(self.weight, self.scale, out, ctx)
            return ops.embed_pairs(self.weight, self.scale, out, ctx, pairs=p.weight, buckets=p.buckets,
                                   mul_prev=p.mul_prev, mul_cur=p.mul_cur, last_token=cache.state)
        ops.embed_rows(self.weight, tokens[:n_rows], out)
        if self.norm is None:
            return out
        return ops.add_rmsnorm(out, None, self.norm.weight, self.norm.eps, torch.empty_like(out), n_rows=n_rows)


class VocabHead(Part):
    def __init__(self, opts: BuildOptions, vocab: int, width: int, name: str,
                 tied_to: TokenEmbedding | None = None, weight_suffix: str = ".weight"):
        self.opts, self.vocab, self.width, self.name = opts, int(vocab), int(width), name
        self.tied_to, self.weight_suffix = tied_to, weight_suffix
        self.proj = Linear(opts, width, [(name, vocab)], out_dtype=torch.float32, weight_suffix=weight_suffix)

    def children(self):
        return [] if self.tied_to is not None else [self.proj]

    def own_param_specs(self):
        if self.tied_to is not None:   # declared so that a stray stored head is reported, not ignored
            return [ParamSpec(f"{self.name}{self.weight_suffix}", (self.vocab, self.width), "matrix", absent=True)]
        return []

    def load_own(self, fetch):
        pass

    def forward(self, h: torch.Tensor, n_rows: int | None = None) -> torch.Tensor:
        if self.tied_to is not None and self.proj.weight is not self.tied_to.weight:
            self.proj.share_weight(self.tied_to.weight)
        return self.proj.forward(h, n_rows=n_rows)
