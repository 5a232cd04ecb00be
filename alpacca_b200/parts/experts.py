"""A feed-forward of routed experts with a grouped router.

    z = W_r h (32-bit);  s = softmax(z) over all experts
    the experts form `groups` equal groups of neighbours; a group's score is its largest s; only experts of the
    `keep` best groups can be chosen; the `top` largest s among them are chosen
    weights = chosen s / (their sum + 1e-20) * scale;  output = sum of weight * expert(h)
    expert(h) = W_down act(W_up h), no biases

Options: `router_bias` (a bias on the logits, tensor `<router>.b`); `gate_name`: gated experts,
expert(h) = W_down (act(W_gate h) * (W_up h)).  With one group, all of it kept and scale 1 the weights are the
softmax over the chosen logits alone (exp(z_j) / sum over the chosen of exp(z)), which is the router of designs that
choose by logit.

`score` "sigmoid" (or "logit"): s = sigmoid(z) (or z) instead of the softmax; `correction` names a tensor [experts]
that is added to s for the CHOICE alone (groups and experts are chosen by s + correction, the weights are the chosen
s); `group_top`: a group's score is the sum of that many of its largest choice scores; `renorm` off: the weights are
not divided by their sum.

The experts' matrices are stacked ([experts, ff, width] and, side by side, [width, experts, ff]) so that a
kernel picks an expert by index from device memory: routing never reaches the host, and a step with routed
experts is captured in a CUDA graph like any other (csrc/moe.cu).  Steps of few tokens read the chosen
experts' rows per (token, expert) pair; steps of many tokens run all experts in two library products with the
weights of experts that were not chosen set to zero (`ops.moe_experts`).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, FeedForward


class RoutedExperts(FeedForward):
    def __init__(self, opts: BuildOptions, width: int, inner: int, n_experts: int, top: int, groups: int, keep: int,
                 scale: float, prefix: str, activation: str = "gelu", router_name: str = "router",
                 expert_names=("e{}.up", "e{}.down"), router_bias: bool = False, gate_name: str | None = None,
                 score: str = "softmax", correction: str | None = None, group_top: int = 1, renorm: bool = True):
        if activation not in ops.MOE_ACTIVATIONS:
            raise ValueError(f"activation must be one of {tuple(ops.MOE_ACTIVATIONS)}, got {activation!r}")
        if n_experts % groups or not 0 < keep <= groups or not 0 < top <= keep * (n_experts // groups):
            raise ValueError(f"{n_experts} experts in {groups} groups, {keep} kept, {top} chosen cannot be routed")
        self.opts, self.width, self.inner, self.E = opts, int(width), int(inner), int(n_experts)
        self.top, self.groups, self.keep, self.scale = int(top), int(groups), int(keep), float(scale)
        self.prefix, self.activation, self.router_name, self.expert_names = prefix, activation, router_name, expert_names
        self.router_bias, self.gate_name = bool(router_bias), gate_name
        if score not in ops.MOE_SCORES or (score == "softmax" and (correction or group_top != 1 or not renorm)):
            raise ValueError(f"{prefix}: score {score!r} with correction {correction!r}, group_top {group_top}, renorm "
                             f"{renorm} is not a router of this part")
        self.score, self.correction_name, self.group_top, self.renorm = score, correction, int(group_top), bool(renorm)
        self.correction = None
        self.router = self.bias = self.w_up = self.w_down = self.w_gate_up = None

    def own_param_specs(self):
        up, down = self.expert_names
        specs = [ParamSpec(f"{self.prefix}.{self.router_name}", (self.E, self.width), "vector", "normal")]
        for e in range(self.E):
            specs.append(ParamSpec(f"{self.prefix}.{up.format(e)}", (self.inner, self.width), "matrix", "normal"))
            specs.append(ParamSpec(f"{self.prefix}.{down.format(e)}", (self.width, self.inner), "matrix", "normal"))
        if self.gate_name is not None:
            specs += [ParamSpec(f"{self.prefix}.{self.gate_name.format(e)}", (self.inner, self.width), "matrix", "normal")
                      for e in range(self.E)]
        if self.router_bias:
            specs.append(ParamSpec(f"{self.prefix}.{self.router_name}.b", (self.E,), "vector", "normal"))
        if self.correction_name is not None:
            specs.append(ParamSpec(f"{self.prefix}.{self.correction_name}", (self.E,), "vector", "normal"))
        return specs

    def load_own(self, fetch):
        specs = self.own_param_specs()
        self.router = fetch(specs[0])
        ups = [fetch(s) for s in specs[1:1 + 2 * self.E:2]]
        self.w_down = torch.stack([fetch(s) for s in specs[2:2 + 2 * self.E:2]], dim=1).contiguous()      # [width, E, ff]
        if self.gate_name is not None:
            gates = [fetch(s) for s in specs[1 + 2 * self.E:1 + 3 * self.E]]
            self.w_gate_up = torch.stack([torch.stack(gates), torch.stack(ups)]).contiguous()      # [2, E, ff, width]
            self.w_up = self.w_gate_up[1]
        else:
            self.w_up = torch.stack(ups).contiguous()
        if self.router_bias:
            self.bias = fetch(specs[1 + (3 if self.gate_name is not None else 2) * self.E])
        if self.correction_name is not None:
            self.correction = fetch(specs[-1])

    def forward(self, h, ctx):
        T = ctx.n_tokens
        idx, wts = ops.moe_route(h, self.router, T, self.groups, self.keep, self.top, self.scale, bias=self.bias,
                                 score=self.score, correction=self.correction, group_top=self.group_top,
                                 renorm=self.renorm)
        out = torch.empty((h.shape[0], self.width), dtype=h.dtype, device=h.device)
        return ops.moe_experts(h, self.w_up, self.w_down, idx, wts, out, T, self.activation, gate_up=self.w_gate_up)
