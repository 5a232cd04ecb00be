"""How a layer arranges its parts: pre-norm, two residual adds
(x += Mixer(Norm1(x)); x += FeedForward(Norm2(x)), alpacca/model.py:486-514).

The residual stream is float32 in memory in both precisions.  A sub-layer's
output is not added at once: it waits in `stream.delta` and is added by the
next norm's fused kernel (which reads the stream anyway).  In steps of a few
rows the norm has no kernel at all where the parts on both sides can share its
work (`OwedNorm` in base.py): the sub-layer adds its output to the residual
itself and hands `stream.owed` to the next reader.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from .base import Block, FeedForward, HalfSum, Mixer, Norm, OwedNorm, WeightedSum
from .layer_norm import LayerNorm


@dataclass
class HiddenStream:
    residual: torch.Tensor            # float32 [T, E]
    delta: torch.Tensor | None = None  # output of the last sub-layer, not yet added
    owed: OwedNorm | None = None       # or: the residual is up to date and these rows stand for `owed.norm`
    next_norm: Norm | None = None      # set by the model: the norm that reads the stream after this block,
                                       # if its reader accepts an OwedNorm in this step
    next_plain: Norm | None = None     # set by the model: the next block's first norm, if that block takes the
                                       # norm's finished output from the block before it (`ready`)
    ready: tuple | None = None         # (norm, rows): the residual is up to date and `rows` are norm(residual)


class PreNormBlock(Block):
    """`after`: a part that acts on the stream once the sub-layers are done (`forward(stream, ctx)`; a layer's
    token input, say).  It reads the stream as it stands, so the last sub-layer's output is not prepared
    for the next block's norm then; if the part has a `cast` (a norm-like stand-in for "the stream in the
    activation dtype"), the last sub-layer may prepare that instead."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None, ffn: FeedForward | None, after=None):
        self.norm1, self.mixer, self.norm2, self.ffn, self.after = norm1, mixer, norm2, ffn, after

    def first_norm(self, n_rows: int) -> Norm | None:
        """The norm that reads the stream when this block starts, if in a step of `n_rows` rows the
        block accepts an `OwedNorm` for it from whatever ran before."""
        if _accepts(self.mixer, n_rows) and self.norm1.deferred() is not None:
            return self.norm1
        return None

    def forward(self, stream: HiddenStream, ctx, cache, write_cache: bool = True) -> None:
        next_norm, stream.next_norm = stream.next_norm, None
        if self.after is not None:
            next_norm = getattr(self.after, "cast", None)
        h = _normed(self.norm1, stream)
        if self.ffn is None:
            _sublayer(stream, next_norm, self.mixer, h, ctx, cache, write_cache)
        else:
            after_mixer = self.norm2 if _accepts(self.ffn, ctx.n_tokens) else None
            _sublayer(stream, after_mixer, self.mixer, h, ctx, cache, write_cache)
            h = _normed(self.norm2, stream)
            _sublayer(stream, next_norm, self.ffn, h, ctx)
        if self.after is not None:
            self.after.forward(stream, ctx)


class ParallelBlock(Block):
    """One norm, both sub-layers read its output: h = Norm(x); x += Mixer(h) + FeedForward(h).
    The stream is float32: the mixer's output is added to it at once and the feed-forward's waits for the
    next norm's kernel, so neither the sum of the two nor the stream is rounded to the activation dtype."""

    def __init__(self, norm: Norm, mixer: Mixer, ffn: FeedForward | None):
        self.norm1, self.mixer, self.ffn = norm, mixer, ffn

    def forward(self, stream: HiddenStream, ctx, cache, write_cache: bool = True) -> None:
        stream.next_norm = None
        h = _normed(self.norm1, stream)
        stream.delta = self.mixer.forward(h, ctx, cache, write_cache)
        if self.ffn is None:
            return
        ops.residual_add(stream.residual, stream.delta, n_rows=ctx.n_tokens)
        stream.delta = self.ffn.forward(h, ctx)


class SandwichBlock(Block):
    """A norm before AND after each sub-layer: x += Post1(Mixer(Norm1(x))); x += Post2(FeedForward(Norm2(x))).

    The norm after a sub-layer acts on the sub-layer's output alone, so that output cannot wait to be added by
    the next norm's kernel as it is: one kernel norms it, adds it to the float32 stream and, between the two
    sub-layers, leaves the next norm's output as well (`ops.post_norm_add`).  A mixer may return a `HalfSum`
    (two mixers side by side whose normed outputs are averaged); the same kernel forms it.  The norms are
    `RMSNorm`s (weight per column, eps), 32-bit arithmetic.  Where the next block is of this kind too, the kernel
    after this block's last sub-layer leaves that block's first norm as well (`first_plain_norm`,
    `HiddenStream.ready`).

    With `LayerNorm`s (weight and bias, centred) the same arrangement runs `ops.post_layer_norm_add`; then
    `residual_mult` m scales what joins the stream, x += m * Post(Sublayer(Norm(x))), and two mixers side by side
    may hand over a `WeightedSum` (c_left * left + c_right * right)."""

    def __init__(self, norm1: Norm, mixer: Mixer, post1: Norm, norm2: Norm | None = None,
                 ffn: FeedForward | None = None, post2: Norm | None = None, residual_mult: float = 1.0):
        if (ffn is None) != (norm2 is None) or (ffn is None) != (post2 is None):
            raise ValueError("a feed-forward comes with a norm before and a norm after it")
        self.residual_mult = float(residual_mult)
        if self.residual_mult != 1.0 and not all(isinstance(n, LayerNorm) for n in (post1, post2) if n is not None):
            raise ValueError("a factor on what joins the stream comes with layer norms after the sub-layers "
                             "(an RMS norm takes it into its weight: `RMSNorm(scale=)`)")
        self.norm1, self.mixer, self.post1 = norm1, mixer, post1
        self.norm2, self.ffn, self.post2 = norm2, ffn, post2

    def cache_specs(self) -> list:
        several = getattr(self.mixer, "cache_specs", None)      # mixers side by side, a mixer with two states: an entry for each
        if several is not None:
            return several()
        return super().cache_specs()

    def first_plain_norm(self):
        """The norm whose finished output this block takes from the kernel that ended the block before it."""
        return self.norm1

    def forward(self, stream: HiddenStream, ctx, cache, write_cache: bool = True) -> None:
        stream.next_norm = None
        after, stream.next_plain = stream.next_plain, None
        ready, stream.ready = stream.ready, None
        if ready is not None and ready[0] is self.norm1:
            h = ready[1]
        else:
            h = _normed(self.norm1, stream)
        stream.delta = None
        y = self.mixer.forward(h, ctx, cache, write_cache)
        last = self.post1 if self.ffn is None else self.post2
        if after is not None and not (hasattr(after, "weight") and getattr(after, "eps", None) == last.eps
                                      and isinstance(after, LayerNorm) == isinstance(last, LayerNorm)):
            after = None
        if self.ffn is not None:
            h = _post_add(self.post1, stream.residual, y, ctx, then=self.norm2, mult=self.residual_mult)
            y = self.ffn.forward(h, ctx)
        rows = _post_add(last, stream.residual, y, ctx, then=after, mult=self.residual_mult)
        if after is not None:
            stream.ready = (after, rows)


def _post_add(post: Norm, residual, y, ctx, then: Norm | None = None, mult: float = 1.0):
    """residual += mult * post(y); returns then(residual) in the activation dtype where `then` is given."""
    out = None
    if then is not None:
        out = torch.empty((residual.shape[0], residual.shape[-1]), dtype=then.opts.dtype, device=residual.device)
    if isinstance(post, LayerNorm):
        if then is not None and (not isinstance(then, LayerNorm) or then.eps != post.eps):
            raise ValueError("the norm after a sub-layer and the norm that reads the stream next are of one kind and eps")
        more = {}
        if isinstance(y, WeightedSum):
            more = {"b": y.b, "ca": y.ca, "cb": y.cb}
            y = y.a
        elif isinstance(y, HalfSum):
            raise ValueError("a half sum of normed outputs is formed before an RMS norm, not before a layer norm")
        return ops.post_layer_norm_add(residual, y, post.weight, post.bias, post.eps, mult, ctx,
                                       next_weight=then.weight if then else None,
                                       next_bias=then.bias if then else None, out=out, **more)
    if isinstance(y, WeightedSum) or mult != 1.0:
        raise ValueError("a weighted sum of two mixers and a factor on the stream's addition come with layer norms")
    more = {}
    if isinstance(y, HalfSum):
        more = {"b": y.b, "wa": y.wa, "wb": y.wb}
        if y.eps != post.eps:
            raise ValueError("the norms of a sum of two mixers and the norm after it share one eps")
        y = y.a
    return ops.post_norm_add(residual, y, post.weight, post.eps, ctx, next_weight=then.weight if then else None,
                             out=out, **more)


def _accepts(part, n_rows: int) -> bool:
    accepts = getattr(part, "accepts_owed_norm", None)
    return bool(accepts(n_rows)) if accepts is not None else False


def _normed(norm: Norm, stream: HiddenStream):
    """What `norm` gives its reader: the rows prepared for it, or its own kernel's output."""
    if stream.owed is not None:
        owed, stream.owed = stream.owed, None
        if owed.norm is not norm:
            raise RuntimeError("rows were prepared for another norm than the one that reads them")
        return owed
    return norm.forward(stream.residual, stream.delta)


def _sublayer(stream: HiddenStream, then_norm: Norm | None, part, h, *args) -> None:
    """Runs a mixer or feed-forward; its output waits in `stream.delta`, or, where the part and the
    norm after it allow, is added by the part itself and prepared for that norm (`stream.owed`)."""
    if (then_norm is not None and getattr(part, "adds_to_residual", False)
            and then_norm.deferred() is not None):
        out = part.forward(h, *args, then=(stream.residual, then_norm))
    else:
        out = part.forward(h, *args)
    if isinstance(out, OwedNorm):
        stream.owed, stream.delta = out, None
    else:
        stream.delta = out
