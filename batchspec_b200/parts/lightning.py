"""Lightning attention: linear attention whose state per request and head is a [key dim x value dim] matrix S that
decays by a fixed factor per head.

With h the token's normed input and H heads:

    q, k = silu(Wq h), silu(Wk h)   (H x dim),   v = silu(Wv h)   (H x v_dim)
    S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t                 the read-out sees the token's own write
    out = Wo (concat_heads(o) / rms(concat_heads(o)) * w * sigmoid(Wg h))    one RMS norm over all heads together

Everything after the projections is float32: silu, the recurrence, its state and the output norm.  The state of a
request is one float32 row [S of every head], zero at admission.  Launch sequence: one product for [Wq; Wk; Wv; Wg]
with float32 output -> lightning_recurrence -> gated_rmsnorm (sigmoid gate, one group) -> output projection."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import MIXERS, Mixer, ParamSpec, Runtime, StateSpec, register_part


@register_part(MIXERS, "lightning_attention")
class LightningAttention(Mixer):
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, n_heads: int, head_dim: int, v_dim: int, decay: Sequence[float],
                 eps: float):
        if n_heads <= 0 or not 0 < head_dim <= 256 or v_dim <= 0:
            raise ValueError(f"the lightning attention kernel takes key sizes up to 256, got {head_dim}")
        if len(decay) != n_heads:
            raise ValueError(f"{n_heads} heads need {n_heads} decay factors, got {len(decay)}")
        self.runtime = runtime
        self.dim, self.n_heads, self.head_dim, self.v_dim = int(dim), int(n_heads), int(head_dim), int(v_dim)
        self.eps = float(eps)
        self.decay = torch.tensor([float(x) for x in decay], dtype=torch.float32, device=runtime.device)

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, v = self.n_heads * self.head_dim, self.n_heads * self.v_dim
        return {"q": ParamSpec((qk, self.dim)), "k": ParamSpec((qk, self.dim)), "v": ParamSpec((v, self.dim)),
                "g": ParamSpec((v, self.dim)), "norm": ParamSpec((v,), role="vector", init="ones_normal"),
                "o": ParamSpec((self.dim, v))}

    def bind(self, params):
        ops.require("state_mixers")
        self.w_in = torch.cat([params[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.norm = params["norm"].to(torch.float32).contiguous()
        self.w_o = params["o"].contiguous()
        qk, v = self.n_heads * self.head_dim, self.n_heads * self.v_dim
        self.k_off, self.v_off, self.g_off = qk, 2 * qk, 2 * qk + v

    def state_spec(self) -> StateSpec:
        return StateSpec((self.n_heads * self.v_dim * self.head_dim,), torch.float32)

    def forward(self, x, ctx, cache):
        H, dk, dv = self.n_heads, self.head_dim, self.v_dim
        with bucket("lightning.in_proj"):
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        with bucket("lightning.recurrence"):
            o = ops.lightning_recurrence(proj, 0, self.k_off, self.v_off, self.decay, cache.state, ctx, H, dk, dv)
        with bucket("lightning.out_norm"):
            y = ops.gated_rmsnorm(o, proj[:, self.g_off:self.g_off + H * dv], self.norm, self.eps, 1, H * dv, x.dtype,
                                  gate_act="sigmoid")
        with bucket("lightning.o_proj"):
            return ops.linear(y, self.w_o)
