"""Selective scan (the Mamba mixer): a diagonal recurrent state per channel whose step, input and read-out vectors
depend on the token.

With h the token's normed input, ``inner`` channels, ``n_state`` states per channel, ``dt_rank`` and ``taps``:

    [x | z] = W_in h
    x <- silu(conv(x) + conv_bias)                 causal, per channel, ``taps`` long, the last tap is the token's own
    [dt | B | C] = W_x x;   dt <- softplus(W_dt dt + dt_bias)   one step per channel;   A = -exp(A_log)
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;    y_c = sum_n S[c, n] C_n + D_c x_c
    out = W_o (y * silu(z))

The products run in the run dtype with float32 accumulation; what they feed into the recurrence (x after the
convolution, B, C, the raw step) leaves them in float32, and softplus, the exponentials, the state and the gate are
float32.  State of a request: one float32 row [S as [n_state, inner] | the convolution's last taps-1 inputs].  Launch
sequence: in-projection (float32 out) -> scan_conv -> three small products (dt part in the run dtype, [B | C] in
float32, the raw step in float32) -> selective_scan -> output projection.  ``pre_projection`` is everything before the
output projection."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import MIXERS, Mixer, ParamSpec, Runtime, StateSpec, register_part


@register_part(MIXERS, "selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, inner: int, n_state: int, dt_rank: int, taps: int):
        if inner <= 0 or not 0 < n_state <= 256 or dt_rank <= 0 or taps < 1:
            raise ValueError(f"the selective scan kernel takes up to 256 states per channel, got {n_state}")
        self.runtime = runtime
        self.dim, self.inner, self.n_state = int(dim), int(inner), int(n_state)
        self.dt_rank, self.taps = int(dt_rank), int(taps)
        self.tail_off = self.n_state * self.inner

    def param_specs(self) -> Dict[str, ParamSpec]:
        I, N, R = self.inner, self.n_state, self.dt_rank
        return {"in": ParamSpec((2 * I, self.dim)), "conv": ParamSpec((I, self.taps)),
                "conv_bias": ParamSpec((I,), role="vector"), "x": ParamSpec((R + 2 * N, I)), "dt": ParamSpec((I, R)),
                "dt_bias": ParamSpec((I,), role="vector"), "A_log": ParamSpec((I, N)),
                "D": ParamSpec((I,), role="vector", init="ones_normal"), "o": ParamSpec((self.dim, I))}

    def bind(self, params):
        ops.require("state_mixers")
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.w_in, self.wo = params["in"].contiguous(), params["o"].contiguous()
        self.conv, self.conv_bias = f32(params["conv"]), f32(params["conv_bias"])
        self.w_x_dt = params["x"][:self.dt_rank].contiguous()
        self.w_x_bc = params["x"][self.dt_rank:].contiguous()
        self.w_dt = params["dt"].contiguous()
        self.dt_bias, self.a_log, self.d_skip = f32(params["dt_bias"]), f32(params["A_log"]), f32(params["D"])
        self.decay_table = ops.scan_decay_table(self.a_log)     # A = -exp(A_log) as [N, inner], read by the scan kernel

    @property
    def out_width(self) -> int:
        return self.inner

    def state_spec(self) -> StateSpec:
        return StateSpec((self.tail_off + (self.taps - 1) * self.inner,), torch.float32)

    def forward(self, x, ctx, cache):
        y = self.pre_projection(x, ctx, cache)
        with bucket("scan.o_proj"):
            return ops.linear(y, self.wo)

    def pre_projection(self, x, ctx, cache, out=None, out_scale: float = 1.0):
        """y * silu(z) [n, inner] in the run dtype, times ``out_scale``; written into ``out`` (a view of columns of
        wider rows) when given."""
        n = x.shape[0]
        if out is None:
            out = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        with bucket("scan.in_proj"):
            xz = ops.linear(x, self.w_in, out_dtype=torch.float32)
        with bucket("scan.conv"):
            xc, xr = ops.scan_conv(xz, self.conv, self.conv_bias, cache.state, self.tail_off, ctx, self.inner,
                                   self.taps, x.dtype)
        with bucket("scan.x_proj"):
            dt_low = ops.linear(xr, self.w_x_dt)
            bc = ops.linear(xr, self.w_x_bc, out_dtype=torch.float32)
            dt_raw = ops.linear(dt_low, self.w_dt, out_dtype=torch.float32)
        with bucket("scan.recurrence"):
            ops.selective_scan(xz, xc, dt_raw, bc, self.a_log, self.d_skip, self.dt_bias, cache.state, self.tail_off,
                               ctx, out, out_scale, self.inner, self.n_state, self.taps, self.decay_table)
        return out
