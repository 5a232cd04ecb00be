"""The Mavidra decoder, put together from the parts.

The embedded tokens are scaled and a row of a hashed table of (previous token, token) pairs is added; then the layers as
config.json lists them, each with a layer norm (weight and bias) before and after each sub-layer and a factor m on what
joins the stream: x += m * norm1b(mixer(norm1(x))); x += m * norm2b(ff(norm2(x))) where the layer has a feed-forward.
A layer's mixer is gated linear attention (a decay per key channel and token), latent attention with a sliding
window and a gate per head (a layer may read the latent rows that an earlier layer caches), or two mixers side by
side whose outputs are added with constant weights: grouped attention with query/key norm, a rotation in halves, a
sink and a gate per head, beside the gated delta rule with short convolutions.  The feed-forward is routed experts
(gated, SiLU) with sigmoid scores, a correction that acts on the choice alone, groups scored by their two best
members, and weights that are not renormalised.  The head is the embedding table itself (without its factor).

Tensor names (matrices [out, in], named by their prefix alone; a norm `n` has weight `n` and bias `n.b`):
    embed, bigram, final.norm, l<i>.norm1, l<i>.norm1b, l<i>.norm2, l<i>.norm2b
    l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}                                              gla
    l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}                                   latent_attention (no dkv* with kv_from)
    l<i>.mix.left.{q,k,v,q.norm,k.norm,sink,g,o}
    l<i>.mix.right.{q,k,v,q.conv,k.conv,v.conv,b,a,A_log,dt_bias,norm,g,o}            parallel
    l<i>.mlp.router, l<i>.mlp.correction, l<i>.mlp.e<j>.{gate,up,down}
"""
from __future__ import annotations

import torch

from ..config.mavidra import MavidraConfig
from ..config.registry import register_architecture
from ..engine.model import DecoderSpec, Run
from ..parts import (BuildOptions, GatedDeltaRule, GatedLinearAttention, LatentAttention, LayerNorm, MapsAttention,
                     PairTable, RotaryEncoding, RoutedExperts, SandwichBlock, SideBySide, TokenEmbedding, VocabHead)

GROUP_TOP = 2        # a group of experts is scored by the sum of its two largest choice scores


@register_architecture("Mavidra", MavidraConfig)
def build_mavidra(cfg: MavidraConfig, opts: BuildOptions) -> DecoderSpec:
    E, eps = cfg.width, cfg.eps
    rotations: dict = {}          # layers with the same rotation share one table

    def norm(name):
        return LayerNorm(opts, E, eps, name, weight_suffix="", bias_suffix=".b")

    def rotation(dim, rot, pairing):
        if rot["dims"] == 0:          # nothing is rotated
            return None
        key = (dim, rot["dims"], float(rot["base"]), pairing)
        if key not in rotations:
            rotations[key] = RotaryEncoding(opts, dim, rot["dims"], float(rot["base"]), pairing)
        return rotations[key]

    def window(mx):
        return mx["mask"]["size"] if mx.get("mask") else None

    # a latent-attention layer's cache serves the widest window among itself and the layers that read it
    keeps: dict = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "latent_attention":
            owner = layer["mixer"].get("kv_from")
            owner = i if owner is None else owner
            w = window(layer["mixer"])
            keeps[owner] = "all" if w is None or keeps.get(owner) == "all" else max(w, keeps.get(owner, 0))

    layers, schedule, run_of_layer = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}", layer["mixer"]
        reads = None
        # the mixers' outputs are normed right away: they leave their last product in float32
        if layer["type"] == "gla":
            if "rank" not in mx:
                raise ValueError(f"layers[{i}].mixer: the decay projection's inner size `rank` is neither in the "
                                 "configuration nor given by a checkpoint's tensor shapes")
            mixer = GatedLinearAttention(opts, E, mx["heads"], mx["dim"], mx["vdim"], mx["rank"], mx["tau"], eps,
                                         f"{p}.mix", out_dtype=torch.float32)
        elif layer["type"] == "latent_attention":
            owner = mx.get("kv_from")
            reads = run_of_layer[owner] if owner is not None else None
            mixer = LatentAttention(opts, E, mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["q_rank"],
                                    mx["kv_rank"], mx["scale"], eps, rotation(mx["rot_dim"], mx["rot"], "llama"),
                                    f"{p}.mix", sink=False, window=window(mx), keep_window=keeps[i if owner is None else owner],
                                    head_gate="g", own_kv=owner is None, out_dtype=torch.float32)
        else:
            lf, rt = mx["left"], mx["right"]
            left = MapsAttention(opts, E, lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"],
                                 rotation(lf["dim"], lf["rot"], "neox"), f"{p}.mix.left", lf["scale"], eps, qk_norm=True,
                                 sink=True, head_gate="g", out_dtype=torch.float32)
            right = GatedDeltaRule(opts, E, rt["heads"], rt["kv_heads"], rt["dim"], rt["vdim"], rt["conv"], eps,
                                   f"{p}.mix.right", out_dtype=torch.float32)
            mixer = SideBySide(opts, E, left, right, eps, f"{p}.mix", scales=(mx["left_scale"], mx["right_scale"]))
        run_of_layer[i] = len(schedule)
        schedule.append(Run(i, reads_entry_of=reads))
        mlp = layer.get("mlp")
        if mlp is None:
            layers.append(SandwichBlock(norm(f"{p}.norm1"), mixer, norm(f"{p}.norm1b"), residual_mult=cfg.residual_mult))
            continue
        rt = mlp["router"]
        groups = rt.get("groups") or {"count": 1, "keep": 1}
        ffn = RoutedExperts(opts, E, mlp["expert"]["ff"], rt["experts"], rt["top"], groups["count"], groups["keep"], 1.0,
                            f"{p}.mlp", activation="silu", gate_name="e{}.gate", score="sigmoid",
                            correction="correction", group_top=GROUP_TOP, renorm=False)
        layers.append(SandwichBlock(norm(f"{p}.norm1"), mixer, norm(f"{p}.norm1b"), norm(f"{p}.norm2"), ffn,
                                    norm(f"{p}.norm2b"), residual_mult=cfg.residual_mult))
    emb = cfg.embedding
    pairs = None
    if emb.get("bigram") is not None:
        bg = emb["bigram"]
        pairs = PairTable(opts, bg["buckets"], E, bg["mul_prev"], bg["mul_cur"], "bigram")
    embedding = TokenEmbedding(opts, cfg.vocab, E, "embed", weight_suffix="", scale=float(emb["scale"]), pairs=pairs)
    return DecoderSpec(
        embedding=embedding, layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=VocabHead(opts, cfg.vocab, E, "head", tied_to=embedding, weight_suffix=""),
        stop_token_ids=cfg.stop_tokens, vocab_size=cfg.vocab)
