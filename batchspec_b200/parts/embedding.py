"""Parts that add to the embedding rows."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import INPUT_PARTS, InputPart, ParamSpec, Runtime, StateSpec, register_part


@register_part(INPUT_PARTS, "bigram_hash")
class BigramHash(InputPart):
    """Adds a row of a hashed bigram table to every token's embedding: row
    (previous token * mul_prev + token * mul_cur) mod buckets, and the table's last row (number ``buckets``) for a
    request's first token.  The previous token of a portion's first token is kept per request (an int32 of state)."""
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, vocab: int, buckets: int, mul_prev: int, mul_cur: int):
        if buckets <= 0 or not (0 <= mul_prev < 2 ** 31 and 0 <= mul_cur < 2 ** 31):
            raise ValueError(f"a hashed table needs at least one bucket and multipliers in [0, 2^31), got {buckets}, "
                             f"{mul_prev}, {mul_cur}")
        self.runtime, self.dim, self.vocab = runtime, int(dim), int(vocab)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.table = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((self.buckets + 1, self.dim))}

    def bind(self, params):
        self.table = params["table"].contiguous()

    def state_spec(self) -> StateSpec:
        return StateSpec((1,), torch.int32)

    def forward(self, resid, ctx, state=None) -> None:
        with bucket("embed"):
            ops.bigram_add(resid, self.table, state, ctx, self.buckets, self.mul_prev, self.mul_cur, self.vocab)
