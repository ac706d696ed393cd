"""Pre-norm residual block (batchspec/models/base_model.py:53-56):
h = x + m mixer(norm1(x));  x' = h + m ffn(norm2(h)), m = ``residual_mult`` (1 unless the design scales its
branches).  The adds are carried as a pending branch output and fused into the following norm kernel; the residual
stream itself is float32.  A block returns its last branch unscaled; ``residual_mult`` is what whoever adds it
multiplies it by (the next block gets it as ``pending_scale``)."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .base import (BLOCKS, BRANCH_SCALES, FEED_FORWARDS, MIXERS, NORMS, STREAM_MIXES, Block, ParamSpec, Part, Runtime,
                   register_part)


@register_part(BLOCKS, "prenorm")
class PreNormBlock(Block):
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "ffn": FEED_FORWARDS}

    def __init__(self, residual_mult: float = 1.0, **parts):
        super().__init__(**parts)
        self.residual_mult = float(residual_mult)

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0, pending_vec=None):
        a = self.norm1.forward(resid, pending, pending_scale, pending_vec)
        y = self.mixer.forward(a, ctx, cache)
        f = self.norm2.forward(resid, y, self.residual_mult)
        return resid, self.ffn.forward(f, ctx)


@register_part(BLOCKS, "prenorm_mixer")
class PreNormMixerBlock(Block):
    """A pre-norm layer without a feed-forward: x' = x + m mixer(norm1(x))."""
    SLOTS = {"norm1": NORMS, "mixer": MIXERS}

    def __init__(self, residual_mult: float = 1.0, **parts):
        super().__init__(**parts)
        self.residual_mult = float(residual_mult)

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0, pending_vec=None):
        a = self.norm1.forward(resid, pending, pending_scale, pending_vec)
        return resid, self.mixer.forward(a, ctx, cache)


@register_part(BRANCH_SCALES, "channel")
class ChannelScale(Part):
    """A learned factor per column on a branch's output before it joins the residual stream (layer scale).  Held in
    float32: the product and the sum are taken there."""
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int):
        self.runtime, self.dim = runtime, int(dim)
        self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), role="vector", init="ones_normal")}

    def bind(self, params):
        self.weight = params["weight"].to(torch.float32).contiguous()


@register_part(BLOCKS, "prenorm_scaled")
class ScaledPreNormBlock(Block):
    """Pre-norm layer whose branches are multiplied column by column by learned vectors before the residual sum:
    h = x + s1 * mixer(norm1(x));  x' = h + s2 * ffn(norm2(h))."""
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "scale1": BRANCH_SCALES, "norm2": NORMS, "ffn": FEED_FORWARDS,
             "scale2": BRANCH_SCALES}

    @property
    def residual_vec(self):
        return self.scale2.weight

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0, pending_vec=None):
        a = self.norm1.forward(resid, pending, pending_scale, pending_vec)
        y = self.mixer.forward(a, ctx, cache)
        f = self.norm2.forward(resid, y, 1.0, self.scale1.weight)
        return resid, self.ffn.forward(f, ctx)


@register_part(BLOCKS, "prenorm_mixer_scaled")
class ScaledPreNormMixerBlock(Block):
    """The same without a feed-forward: x' = x + s1 * mixer(norm1(x))."""
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "scale1": BRANCH_SCALES}

    @property
    def residual_vec(self):
        return self.scale1.weight

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0, pending_vec=None):
        a = self.norm1.forward(resid, pending, pending_scale, pending_vec)
        return resid, self.mixer.forward(a, ctx, cache)


@register_part(STREAM_MIXES, "hyper_connection")
class HyperConnection(Part):
    """The coefficients of one sublayer of a model that keeps ``streams`` copies x_1 .. x_S of the residual per
    token: the sublayer reads u = sum_s in[s] x_s, and its result y joins all streams at once,
    x_t <- sum_s mix[s, t] x_s + out[t] * y.  Held in float32; ``read`` = in, ``write`` = [mix | out] as one table."""
    graph_safe = True

    def __init__(self, runtime: Runtime, streams: int):
        self.runtime, self.streams = runtime, int(streams)
        if not 0 < self.streams <= 16:
            raise ValueError(f"between 1 and 16 residual streams, got {streams}")
        self.read = self.write = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = self.streams
        return {"in": ParamSpec((s,), role="vector", init="ones_normal"),
                "out": ParamSpec((s,), role="vector", init="ones_normal"),
                "mix": ParamSpec((s, s), role="vector", init="ones_normal")}

    def bind(self, params):
        if torch.device(self.runtime.device).type == "cuda":
            ops.require("streams")                # the kernels of csrc/streams.cu
        self.read = params["in"].to(torch.float32).contiguous()
        self.write = torch.cat([params["mix"].to(torch.float32).reshape(-1),
                                params["out"].to(torch.float32).reshape(-1)]).contiguous()


@register_part(BLOCKS, "hyper_prenorm")
class HyperPreNormBlock(Block):
    """Pre-norm layer over several residual streams (hyper-connections), branches multiplied column by column by
    learned vectors: for the mixer and then the feed-forward, u = sum_s in[s] x_s; y = scale * sublayer(norm(u));
    x_t <- sum_s mix[s, t] x_s + out[t] * y.  The join of a branch and the read of the next one ride in the norm's
    kernel; the last branch is returned with its vector and coefficients for whoever comes next.  ``expand_from``
    [n, d]: ``resid`` holds nothing yet (the first run of a step) and every stream starts as this row."""
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "scale1": BRANCH_SCALES, "hc1": STREAM_MIXES, "norm2": NORMS,
             "ffn": FEED_FORWARDS, "scale2": BRANCH_SCALES, "hc2": STREAM_MIXES}

    @property
    def residual_vec(self):
        return self.scale2.weight

    @property
    def residual_mix(self):
        return self.hc2.write

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0, pending_vec=None, pending_mix=None,
                expand_from=None):
        assert pending_scale == 1.0 and (pending is None or pending_mix is not None)
        a = self.norm1.forward_streams(resid, pending, pending_vec, pending_mix, self.hc1.read, expand_from)
        y = self.mixer.forward(a, ctx, cache)
        f = self.norm2.forward_streams(resid, y, self.scale1.weight, self.hc1.write, self.hc2.read)
        return resid, self.ffn.forward(f, ctx)


@register_part(BLOCKS, "hyper_prenorm_mixer")
class HyperPreNormMixerBlock(Block):
    """The same without a feed-forward."""
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "scale1": BRANCH_SCALES, "hc1": STREAM_MIXES}

    @property
    def residual_vec(self):
        return self.scale1.weight

    @property
    def residual_mix(self):
        return self.hc1.write

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0, pending_vec=None, pending_mix=None,
                expand_from=None):
        assert pending_scale == 1.0 and (pending is None or pending_mix is not None)
        a = self.norm1.forward_streams(resid, pending, pending_vec, pending_mix, self.hc1.read, expand_from)
        return resid, self.mixer.forward(a, ctx, cache)
