"""Parts that run on the head's output."""
from __future__ import annotations

from ..kernels import ops
from .base import LOGITS_PARTS, LogitsPart, Runtime, register_part


@register_part(LOGITS_PARTS, "tanh_softcap")
class TanhSoftCap(LogitsPart):
    """logits <- cap * tanh(logits / cap), in place on the float32 logits."""
    graph_safe = True

    def __init__(self, runtime: Runtime, cap: float):
        self.runtime, self.cap = runtime, float(cap)
        if not self.cap > 0:
            raise ValueError(f"a soft cap must be positive, got {cap}")

    def forward(self, logits, ctx) -> None:
        ops.tanh_softcap_(logits, self.cap)


@register_part(LOGITS_PARTS, "scale")
class LogitScale(LogitsPart):
    """logits <- factor * logits, in place on the float32 logits."""
    graph_safe = True

    def __init__(self, runtime: Runtime, factor: float):
        self.runtime, self.factor = runtime, float(factor)

    def forward(self, logits, ctx) -> None:
        if self.factor != 1.0:
            ops.scale_(logits, self.factor)
