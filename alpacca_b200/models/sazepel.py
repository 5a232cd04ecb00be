"""The Sazepel decoder, put together from the parts.

The embedded tokens are normed once; then the layers as config.json lists them, each with a norm before and after
each sub-layer: x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))) where the layer has a feed-forward.  Every
one of these norms has ONE number as its weight.  A layer's mixer is a retention (linear attention with a fixed
decay per head, rotated q and k, a norm per head, a SiLU gate) or two mixers side by side: an attention without
positions whose softmax weights are mixed across heads (query, key and value norms without weights, a sigmoid
gate) beside a retention, averaged after a norm of each over the model width.  The feed-forward is routed experts
(gated, SiLU) whose router has a bias and weighs the chosen experts by the softmax over their logits alone.  The
last norm's weight carries the factor on the logits.

Tensor names (matrices [out, in], named by their prefix alone):
    embed, embed.norm, head, final.norm, l<i>.norm1, l<i>.norm1b, l<i>.norm2, l<i>.norm2b
    l<i>.mix.{q,k,v,g,o}                                         retention
    l<i>.mix.left.{q,k,v,talk,g,o}, l<i>.mix.right.{q,k,v,g,o}, l<i>.mix.left.out, l<i>.mix.right.out     parallel
    l<i>.mlp.router, l<i>.mlp.router.b, l<i>.mlp.e<j>.{gate,up,down}
"""
from __future__ import annotations

import torch

from ..config.registry import register_architecture
from ..config.sazepel import SazepelConfig
from ..engine.model import DecoderSpec
from ..parts import (BuildOptions, DecayLinearAttention, MapsAttention, RMSNorm, RotaryEncoding, RoutedExperts,
                     SandwichBlock, SideBySide, TokenEmbedding, VocabHead)


@register_architecture("Sazepel", SazepelConfig)
def build_sazepel(cfg: SazepelConfig, opts: BuildOptions) -> DecoderSpec:
    E, eps = cfg.width, cfg.eps
    rotations: dict = {}          # layers with the same rotation share one table

    def norm(name, scale=1.0):
        return RMSNorm(opts, E, eps, name, weight_suffix="", scalar=True, scale=scale)

    def rotation(dim, rot):
        if rot["dims"] == 0:          # nothing is rotated
            return None
        key = (dim, rot["dims"], float(rot["base"]))
        if key not in rotations:
            rotations[key] = RotaryEncoding(opts, dim, rot["dims"], float(rot["base"]), "neox")
        return rotations[key]

    def retention(mx, prefix):
        # the mixers' outputs are normed right away: they leave their last product in float32
        return DecayLinearAttention(opts, E, mx["heads"], mx["dim"], mx["vdim"], mx["decay"], eps, prefix,
                                    activation=None, position=rotation(mx["dim"], mx["rot"]),
                                    key_scale=float(mx["dim"]) ** -0.5, head_norm=True, norm_weight=False,
                                    gate="silu", out_dtype=torch.float32)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}", layer["mixer"]
        if layer["type"] == "retention":
            mixer = retention(mx, f"{p}.mix")
        else:
            lf = mx["left"]
            left = MapsAttention(opts, E, lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"], None, f"{p}.mix.left",
                                 lf["scale"], eps, qk_norm=True, qk_norm_weight=False, value_norm=True,
                                 head_mix="talk", gate="g", out_dtype=torch.float32)
            mixer = SideBySide(opts, E, left, retention(mx["right"], f"{p}.mix.right"), eps, f"{p}.mix")
        mlp = layer.get("mlp")
        if mlp is None:
            layers.append(SandwichBlock(norm(f"{p}.norm1"), mixer, norm(f"{p}.norm1b")))
            continue
        rt = mlp["router"]
        ffn = RoutedExperts(opts, E, mlp["expert"]["ff"], rt["experts"], rt["top"], 1, 1, 1.0, f"{p}.mlp",
                            activation="silu", router_bias=True, gate_name="e{}.gate")
        layers.append(SandwichBlock(norm(f"{p}.norm1"), mixer, norm(f"{p}.norm1b"), norm(f"{p}.norm2"), ffn,
                                    norm(f"{p}.norm2b")))
    return DecoderSpec(
        embedding=TokenEmbedding(opts, cfg.vocab, E, "embed", weight_suffix="", norm=norm("embed.norm")),
        layers=layers, final_norm=norm("final.norm", scale=float(cfg.logit_scale)),
        head=VocabHead(opts, cfg.vocab, E, "head", weight_suffix=""),
        stop_token_ids=cfg.stop_tokens, vocab_size=cfg.vocab)
