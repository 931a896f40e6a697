"""A feed-forward of routed experts with a grouped router.

    z = W_r h (32-bit);  s = softmax(z) over all experts
    the experts form `groups` equal groups of neighbours; a group's score is its largest s; only experts of the
    `keep` best groups can be chosen; the `top` largest s among them are chosen
    weights = chosen s / (their sum + 1e-20) * scale;  output = sum of weight * expert(h)
    expert(h) = W_down act(W_up h), no biases

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
                 expert_names=("e{}.up", "e{}.down")):
        if activation not in ops.MOE_ACTIVATIONS:
            raise ValueError(f"activation must be one of {tuple(ops.MOE_ACTIVATIONS)}, got {activation!r}")
        if n_experts % groups or not 0 < keep <= groups or not 0 < top <= keep * (n_experts // groups):
            raise ValueError(f"{n_experts} experts in {groups} groups, {keep} kept, {top} chosen cannot be routed")
        self.opts, self.width, self.inner, self.E = opts, int(width), int(inner), int(n_experts)
        self.top, self.groups, self.keep, self.scale = int(top), int(groups), int(keep), float(scale)
        self.prefix, self.activation, self.router_name, self.expert_names = prefix, activation, router_name, expert_names
        self.router = self.w_up = self.w_down = None

    def own_param_specs(self):
        up, down = self.expert_names
        specs = [ParamSpec(f"{self.prefix}.{self.router_name}", (self.E, self.width), "vector", "normal")]
        for e in range(self.E):
            specs.append(ParamSpec(f"{self.prefix}.{up.format(e)}", (self.inner, self.width), "matrix", "normal"))
            specs.append(ParamSpec(f"{self.prefix}.{down.format(e)}", (self.width, self.inner), "matrix", "normal"))
        return specs

    def load_own(self, fetch):
        specs = self.own_param_specs()
        self.router = fetch(specs[0])
        self.w_up = torch.stack([fetch(s) for s in specs[1::2]]).contiguous()
        self.w_down = torch.stack([fetch(s) for s in specs[2::2]], dim=1).contiguous()      # [width, E, ff]

    def forward(self, h, ctx):
        T = ctx.n_tokens
        idx, wts = ops.moe_route(h, self.router, T, self.groups, self.keep, self.top, self.scale)
        out = torch.empty((h.shape[0], self.width), dtype=h.dtype, device=h.device)
        return ops.moe_experts(h, self.w_up, self.w_down, idx, wts, out, T, self.activation)
