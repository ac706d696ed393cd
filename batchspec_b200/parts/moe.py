"""Routed feed-forward (mixture of experts) with sigmoid scores and group-limited choice.

Per token, with h its normed input:  s = sigmoid(Wr h) in float32;  choice = s + correction;  the experts come in
``n_groups`` equal groups of neighbours, a group's score is the sum of its two largest choices, and only experts of
the best ``keep_groups`` groups can be chosen (the others count as minus infinity);  the ``top`` largest choices
are taken;  their weights are s (without the correction) times ``scale``, not renormalised.
Expert e is Wdown_e gelu(Wup_e h) with the exact (erf) GELU and no biases;  the output is the weighted sum.

The experts' matrices are stacked at load ([E, ff, d] and [E, d, ff]); a step sorts its (token, choice) rows by
expert on the device and runs one grouped product per projection over them (``ops.moe_experts``)."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import FEED_FORWARDS, FeedForward, ParamSpec, Runtime, register_part


@register_part(FEED_FORWARDS, "routed_gelu")
class RoutedGelu(FeedForward):
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, intermediate: int, n_experts: int, top: int, scale: float = 1.0,
                 n_groups: int = 1, keep_groups: int = 1, correction: bool = True):
        self.runtime, self.dim, self.intermediate = runtime, int(dim), int(intermediate)
        self.n_experts, self.top, self.scale = int(n_experts), int(top), float(scale)
        self.n_groups, self.keep_groups, self.correction = int(n_groups), int(keep_groups), bool(correction)
        E, G = self.n_experts, self.n_groups
        if not (0 < self.top <= E and G > 0 and E % G == 0 and 0 < self.keep_groups <= G
                and self.keep_groups * (E // G) >= self.top):
            raise ValueError(f"routing of {self.top} of {E} experts in {G} groups keeping {self.keep_groups} is not possible")

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"router": ParamSpec((self.n_experts, self.dim))}
        if self.correction:
            specs["correction"] = ParamSpec((self.n_experts,), role="vector")
        for e in range(self.n_experts):
            specs[f"up{e}"] = ParamSpec((self.intermediate, self.dim))
            specs[f"down{e}"] = ParamSpec((self.dim, self.intermediate))
        return specs

    def bind(self, params):
        if torch.device(self.runtime.device).type == "cuda":
            ops.require("moe")                    # the kernels of csrc/moe.cu
        self.w_router = params["router"].contiguous()
        self.b_correction = params["correction"].contiguous() if self.correction else None
        self.w_up = torch.stack([params[f"up{e}"] for e in range(self.n_experts)]).contiguous()
        self.w_down = torch.stack([params[f"down{e}"] for e in range(self.n_experts)]).contiguous()

    def forward(self, x, ctx):
        with bucket("mlp.router"):
            ids, wts = ops.moe_route(x, self.w_router, self.b_correction, self.n_groups, self.keep_groups, self.top,
                                     self.scale)
        with bucket("mlp.experts"):
            return ops.moe_experts(x, ids, wts, self.w_up, self.w_down, x.dtype)


@register_part(FEED_FORWARDS, "routed_glu")
class RoutedGLU(FeedForward):
    """Routed gated experts with a softmax over the chosen logits: z = Wr h + b in float32; the ``top`` experts of
    largest z are taken and weighted by the softmax over those ``top`` logits alone; expert e is
    Wdown_e (silu(Wgate_e h) * (Wup_e h)), no biases; the output is the weighted sum.  [gate; up] of every expert is
    one stacked matrix, so the first grouped product gives both halves."""
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, intermediate: int, n_experts: int, top: int, bias: bool = True):
        self.runtime, self.dim, self.intermediate = runtime, int(dim), int(intermediate)
        self.n_experts, self.top, self.bias = int(n_experts), int(top), bool(bias)
        if not 0 < self.top <= self.n_experts:
            raise ValueError(f"cannot choose {top} of {n_experts} experts")

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"router": ParamSpec((self.n_experts, self.dim))}
        if self.bias:
            specs["router_bias"] = ParamSpec((self.n_experts,), role="vector")
        for e in range(self.n_experts):
            specs[f"gate{e}"] = ParamSpec((self.intermediate, self.dim))
            specs[f"up{e}"] = ParamSpec((self.intermediate, self.dim))
            specs[f"down{e}"] = ParamSpec((self.dim, self.intermediate))
        return specs

    def bind(self, params):
        if torch.device(self.runtime.device).type == "cuda":
            ops.require("moe")                    # the kernels of csrc/moe.cu
        self.w_router = params["router"].contiguous()
        self.b_router = params["router_bias"].contiguous() if self.bias else None
        self.w_up = torch.stack([torch.cat([params[f"gate{e}"], params[f"up{e}"]], dim=0)
                                 for e in range(self.n_experts)]).contiguous()               # [E, 2 ff, d]
        self.w_down = torch.stack([params[f"down{e}"] for e in range(self.n_experts)]).contiguous()

    def forward(self, x, ctx):
        with bucket("mlp.router"):
            ids, wts = ops.moe_route(x, self.w_router, self.b_router, 1, 1, self.top, 1.0, softmax_top=True)
        with bucket("mlp.experts"):
            return ops.moe_experts(x, ids, wts, self.w_up, self.w_down, x.dtype, glu=True)
