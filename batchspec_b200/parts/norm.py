"""RMSNorm part (batchspec/models/modules/normalization.py:24-39): float32
x * rsqrt(mean(x^2) + eps), cast to the run dtype, then times the weight.
Fused with the residual add that precedes it (base_model.py:53,56).  With ``single_rounding`` the product with the
weight is taken in float32 too and the result is rounded once."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import INPUT_PARTS, NORMS, InputPart, Norm, ParamSpec, Runtime, register_part


@register_part(NORMS, "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    def __init__(self, runtime: Runtime, dim: int, eps: float, single_rounding: bool = False,
                 scalar_weight: bool = False, one_plus: bool = False):
        """``scalar_weight``: the weight is one number (a tensor without dimensions) for all coordinates.
        ``one_plus``: the tensor is stored around zero and the factor is 1 + w (formed once, in float32; the
        product is then float32 with one rounding)."""
        self.runtime, self.dim, self.eps = runtime, int(dim), float(eps)
        self.one_plus = bool(one_plus)
        self.single_rounding = bool(single_rounding) or self.one_plus
        self.scalar_weight = bool(scalar_weight)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec(() if self.scalar_weight else (self.dim,), role="vector",
                                    init="normal" if self.one_plus else "ones_normal")}

    def bind(self, params):
        self.weight = params["weight"].reshape(1).contiguous() if self.scalar_weight else params["weight"]
        if self.one_plus:
            self.weight = (1.0 + self.weight.to(torch.float32)).contiguous()

    def forward(self, resid, delta=None, delta_scale: float = 1.0, delta_vec=None):
        out = torch.empty(resid.shape, dtype=self.runtime.dtype, device=resid.device)
        with bucket("norm"):
            ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, delta_scale, self.single_rounding, delta_vec)
        return out


    def forward_streams(self, streams, delta=None, delta_vec=None, delta_mix=None, read=None, expand=None):
        """For a residual kept as several streams [n, S, d]: ``delta`` (times ``delta_vec`` per column) first joins
        the streams with the coefficients ``delta_mix``; then the rows u = sum_s read[s] x_s are normalised.
        Without ``read`` only the streams are updated.  ``expand`` [n, d]: the streams hold nothing yet and all
        start as this row."""
        n, _, d = streams.shape
        out = torch.empty((n, d), dtype=self.runtime.dtype, device=streams.device) if read is not None else None
        if self.scalar_weight:
            raise ValueError("the norm over several streams takes a weight per column")
        with bucket("norm"):
            ops.stream_norm(streams, delta, delta_vec, delta_mix, read, self.weight, self.eps, out, expand)
        return out


@register_part(NORMS, "layernorm")
class LayerNorm(Norm):
    """Layer norm with weight and bias: (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared
    deviations; float32 arithmetic, fused with the residual add that precedes it."""
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, eps: float):
        self.runtime, self.dim, self.eps = runtime, int(dim), float(eps)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), role="vector", init="ones_normal"),
                "bias": ParamSpec((self.dim,), role="vector")}

    def bind(self, params):
        self.weight, self.bias = params["weight"], params["bias"]
        if self.bias.dtype != self.weight.dtype:
            self.bias = self.bias.to(self.weight.dtype)

    def forward(self, resid, delta=None, delta_scale: float = 1.0, delta_vec=None):
        if delta is not None and (delta_scale != 1.0 or delta_vec is not None):
            ops.residual_update(resid, delta, delta_scale, vec=delta_vec)
            delta = None
        out = torch.empty(resid.shape, dtype=self.runtime.dtype, device=resid.device)
        with bucket("norm"):
            ops.add_layernorm(resid, delta, self.weight, self.bias, self.eps, out)
        return out


@register_part(INPUT_PARTS, "rmsnorm")
class InputRMSNorm(InputPart):
    """RMS norm of the embedding rows, in place on the float32 residual: x / sqrt(mean(x^2) + eps) * w."""
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, eps: float):
        self.runtime, self.dim, self.eps = runtime, int(dim), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), role="vector", init="ones_normal")}

    def bind(self, params):
        self.weight = params["weight"]

    def forward(self, resid, ctx, state=None) -> None:
        out = torch.empty_like(resid)
        with bucket("norm"):
            ops.add_rmsnorm(resid, None, self.weight, self.eps, out, 1.0, True)
        resid.copy_(out)
