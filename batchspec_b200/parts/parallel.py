"""Two mixers side by side on the same input: out = a * left(h) + b * right(h).

Both parts offer ``pre_projection(x, ctx, cache, out, out_scale)`` (everything before their output projection, written
into a view of a shared buffer, already multiplied by its factor), ``out_width`` and ``wo``; the two output projections
then run as one product over the concatenated columns, [a left | b right] [Wo_left | Wo_right]^T, whose float32
accumulation is the sum.  At most one of the two may ask for cache pages and at most one for per-request state; this
mixer passes them on."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import MIXERS, Mixer, ParamSpec, PartSpec, Runtime, build_part, register_part


@register_part(MIXERS, "parallel")
class ParallelMixer(Mixer):
    def __init__(self, runtime: Runtime, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0):
        self.runtime = runtime
        self.left, self.right = build_part(MIXERS, left, runtime), build_part(MIXERS, right, runtime)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        for part in (self.left, self.right):
            if not hasattr(part, "pre_projection"):
                raise ValueError(f"mixer {part.kind!r} cannot run beside another: it has no pre_projection")
        if sum(p.cache_spec() is not None for p in (self.left, self.right)) > 1 or \
                sum(p.state_spec() is not None for p in (self.left, self.right)) > 1:
            raise ValueError("of two mixers side by side at most one may keep cache pages and at most one a state")
        self.position = getattr(self.left, "position", None) or getattr(self.right, "position", None)

    @property
    def graph_safe(self) -> bool:
        return bool(self.left.graph_safe and self.right.graph_safe)

    def param_specs(self) -> Dict[str, ParamSpec]:
        out = {"left." + k: v for k, v in self.left.param_specs().items()}
        out.update({"right." + k: v for k, v in self.right.param_specs().items()})
        return out

    def bind(self, params):
        self.left.bind({k[5:]: v for k, v in params.items() if k.startswith("left.")})
        self.right.bind({k[6:]: v for k, v in params.items() if k.startswith("right.")})
        self.wo = torch.cat([self.left.wo, self.right.wo], dim=1).contiguous()

    def cache_spec(self):
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self):
        return self.left.state_spec() or self.right.state_spec()

    def forward(self, x, ctx, cache):
        n, wl, wr = x.shape[0], self.left.out_width, self.right.out_width
        both = torch.empty((n, wl + wr), dtype=x.dtype, device=x.device)
        self.left.pre_projection(x, ctx, cache, both[:, :wl], self.left_scale)
        self.right.pre_projection(x, ctx, cache, both[:, wl:], self.right_scale)
        with bucket("parallel.o_proj"):
            return ops.linear(both, self.wo)
