"""SwiGLU feed-forward part (batchspec/models/modules/feedforward.py:25-27,62):
u = x W13^T with W13 = [gate; up] fused at load (feedforward.py:35-38),
m = silu(u[:, :I]) * u[:, I:], out = m W2^T.  No biases.  In bfloat16 the fused matrix is stored with gate and up
rows interleaved in groups of 8 (8 gate rows, then their 8 up rows) and decode-sized steps apply the activation inside the product."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import FEED_FORWARDS, FeedForward, ParamSpec, Runtime, register_part


@register_part(FEED_FORWARDS, "swiglu")
class SwiGLU(FeedForward):
    """``activation``: what the gate passes through, "silu" (the reference's), "relu" or "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))."""
    graph_safe = True
    def __init__(self, runtime: Runtime, dim: int, intermediate: int, activation: str = "silu"):
        self.runtime, self.dim, self.intermediate = runtime, int(dim), int(intermediate)
        if activation not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"gated feed-forward activation {activation!r} is not known ({sorted(ops.GATED_ACTIVATIONS)})")
        self.activation = activation
        self.w13 = self.w2 = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate": ParamSpec((self.intermediate, self.dim)),
                "up": ParamSpec((self.intermediate, self.dim)),
                "down": ParamSpec((self.dim, self.intermediate))}

    def bind(self, params):
        # bfloat16: gate and up rows interleaved in groups, so that the GEMM's epilogue can apply the activation
        # (a CTA then holds matching gate and up outputs); float32: the reference's [gate; up] halves
        self.group = ops.GLU_GROUP if (self.runtime.dtype == torch.bfloat16
                                       and self.intermediate % ops.GLU_GROUP == 0) else 0
        if self.group:
            self.w13 = ops.interleave_gate_up(params["gate"], params["up"], self.group)
        else:
            self.w13 = torch.cat([params["gate"], params["up"]], dim=0).contiguous()
        self.w2 = params["down"].contiguous()

    def forward(self, x, ctx):
        if self.group:
            with bucket("mlp.gate_up_proj"):
                m = ops.linear_glu(x, self.w13, self.group, self.activation)
        else:
            with bucket("mlp.gate_up_proj"):
                u = ops.linear(x, self.w13)
            m = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
            with bucket("mlp.act"):
                ops.GATED_ACTIVATIONS[self.activation][1](u, m)
        with bucket("mlp.down_proj"):
            return ops.linear(m, self.w2)


@register_part(FEED_FORWARDS, "clamped_glu")
class ClampedGLU(FeedForward):
    """Gated feed-forward with clamped branches: g = min(Wgate x, limit), u = clamp(Wup x, -limit, limit),
    y = g * sigmoid(alpha * g) * (u + 1), out = Wdown y.  No biases.  [gate; up] is one product."""
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, intermediate: int, limit: float, alpha: float = 1.702):
        self.runtime, self.dim, self.intermediate = runtime, int(dim), int(intermediate)
        self.limit, self.alpha = float(limit), float(alpha)
        self.w13 = self.w2 = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate": ParamSpec((self.intermediate, self.dim)),
                "up": ParamSpec((self.intermediate, self.dim)),
                "down": ParamSpec((self.dim, self.intermediate))}

    def bind(self, params):
        # bfloat16: gate and up rows interleaved in groups, so that the product's epilogue can apply the activation
        # in decode-sized steps; float32: [gate; up] halves
        self.group = ops.GLU_GROUP if (self.runtime.dtype == torch.bfloat16
                                       and self.intermediate % ops.GLU_GROUP == 0) else 0
        if self.group:
            self.w13 = ops.interleave_gate_up(params["gate"], params["up"], self.group)
        else:
            self.w13 = torch.cat([params["gate"], params["up"]], dim=0).contiguous()
        self.w2 = params["down"].contiguous()

    def forward(self, x, ctx):
        if self.group:
            with bucket("mlp.gate_up_proj"):
                m = ops.linear_clamped_glu(x, self.w13, self.alpha, self.limit, self.group)
        else:
            with bucket("mlp.gate_up_proj"):
                u = ops.linear(x, self.w13)
            m = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
            with bucket("mlp.act"):
                ops.clamped_glu(u, m, self.alpha, self.limit)
        with bucket("mlp.down_proj"):
            return ops.linear(m, self.w2)


@register_part(FEED_FORWARDS, "mlp")
class PlainMLP(FeedForward):
    """Two matrices and an activation between them: out = Wdown act(Wup x), no gate and no biases.
    ``activation``: "relu2" (the square of relu) or "gelu" (the exact one).  Decode-sized bfloat16 steps apply the
    square of relu in the first product's epilogue."""
    graph_safe = True
    ACTIVATIONS = ops.PLAIN_ACTIVATIONS

    def __init__(self, runtime: Runtime, dim: int, intermediate: int, activation: str = "relu2"):
        self.runtime, self.dim, self.intermediate = runtime, int(dim), int(intermediate)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"feed-forward activation {activation!r} is not known ({sorted(self.ACTIVATIONS)})")
        self.activation = activation
        self.w1 = self.w2 = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"up": ParamSpec((self.intermediate, self.dim)), "down": ParamSpec((self.dim, self.intermediate))}

    def bind(self, params):
        self.w1, self.w2 = params["up"].contiguous(), params["down"].contiguous()

    def forward(self, x, ctx):
        with bucket("mlp.up_proj"):
            u = ops.linear_act(x, self.w1, self.activation)
        with bucket("mlp.down_proj"):
            return ops.linear(u, self.w2)
