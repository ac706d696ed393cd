"""Grouped-query softmax attention with options that the plain attention part does not have, each a parameter:

* biases on the q, k and v projections (added in float32 to the product's float32 output);
* values of their own size ``v_dim``;
* a position encoding over the first numbers of each head, with a magnitude on cosine and sine (YaRN);
* ``qk_norm_eps``: after the rotation every q and k head is divided by its root mean square (no weight);
  ``qk_norm_weight``: the normalised head is multiplied by a learned weight per number (one for the queries, one for
  the keys, shared by the heads); ``qk_norm_first``: the norm comes before the rotation;
* a mask besides causality: ``chunk`` (a query sees the keys of its own chunk of ``chunk`` positions, counted from
  position 0 of the request) or ``window`` (the last ``window`` keys);
* ``sink``: a learned logit per query head that takes part in the normalisation only:
  out_h(i) = sum_j exp(s_ij) v_j / (exp(sink_h) + sum_j exp(s_ij));  ``fixed_sink``: the same with one given logit for
  all heads and no tensor (0.0 adds one to the denominator);
* ``softcap`` c: a scaled score s becomes c tanh(s / c);
* ``values_are_keys``: there is no value projection, a key as projected is its own value, and only keys are cached;
* ``gate``: the concatenated heads are multiplied element by element by sigmoid(Wg h) before the output projection;
  ``gate="head"``: Wg has one row per head and the head's whole output is multiplied by one number.

Launch sequence: one product for [Wq; Wk; Wv] with float32 output -> q/k/v preparation (bias, rotation, norms, all
float32; q in the run dtype, k and v into their cache pages) -> attention over the pages -> output projection.
``pre_projection`` is everything before the output projection; a mixer that runs this one beside another writes both
results into one buffer and projects them together.
A page holds its keys [kv head, row, head_dim] and then its values [kv head, row, v_dim].  With a chunk mask the
pages that lie wholly before the chunk of the next position are given back."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import (MIXERS, POSITION_ENCODINGS, CacheSpec, Mixer, ParamSpec, PartSpec, Runtime, build_part,
                   register_part)


@register_part(MIXERS, "sink_attention")
class SinkAttention(Mixer):
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 position: PartSpec, v_dim: Optional[int] = None, bias: bool = False,
                 qk_norm_eps: Optional[float] = None, chunk: Optional[int] = None, window: Optional[int] = None,
                 sink: bool = False, fixed_sink: Optional[float] = None, softcap: Optional[float] = None,
                 values_are_keys: bool = False, gate=False, qk_norm_weight: bool = False,
                 qk_norm_first: bool = False):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} must be a positive multiple of n_kv_heads {n_kv_heads}")
        self.runtime = runtime
        self.dim, self.n_heads, self.n_kv_heads, self.head_dim = int(dim), int(n_heads), int(n_kv_heads), int(head_dim)
        self.v_dim = int(v_dim) if v_dim else self.head_dim
        self.values_are_keys, self.gate = bool(values_are_keys), bool(gate)
        self.gate_per_head = gate == "head"
        self.qk_norm_weight, self.qk_norm_first = bool(qk_norm_weight), bool(qk_norm_first)
        if (self.qk_norm_weight or self.qk_norm_first) and not qk_norm_eps:
            raise ValueError("a weight or a place for the q/k norm needs the norm itself (qk_norm_eps)")
        if self.values_are_keys and self.v_dim != self.head_dim:
            raise ValueError(f"values that are the keys have the keys' size {self.head_dim}, not {self.v_dim}")
        self.softcap = float(softcap) if softcap else 0.0
        self.fixed_sink = None if fixed_sink is None else float(fixed_sink)
        if self.softcap < 0 or (sink and fixed_sink is not None):
            raise ValueError("a soft cap is positive; give a learned sink or a fixed one, not both")
        if not (0 < self.head_dim <= 256 and 0 < self.v_dim <= 256):
            raise ValueError(f"attention kernels take head sizes up to 256, got {head_dim} and {self.v_dim}")
        self.scale, self.bias, self.sink = float(scale), bool(bias), bool(sink)
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps else 0.0
        self.chunk, self.window = int(chunk) if chunk else 0, int(window) if window else 0
        if self.chunk < 0 or self.window < 0 or (self.chunk and self.window):
            raise ValueError("give a chunk size or a window, both positive, not both")
        self.position = build_part(POSITION_ENCODINGS, position, runtime)
        self.wqkv = self.wo = self.b = self.sinks = self.sinks_l2 = self.q_norm = self.k_norm = None
        # values that are the keys, at sizes the tensor-core kernels take: those kernels read keys and values from
        # places of their own, so the key rows of the fused product are listed twice and every key is stored as its
        # own value too (twice the pages, tensor-core speed); at other sizes the pages hold keys only
        self.copy_keys = self.values_are_keys and self._tensor_cores(runtime.dtype)

    def param_specs(self) -> Dict[str, ParamSpec]:
        q, k, v = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.n_kv_heads * self.v_dim
        specs = {"q": ParamSpec((q, self.dim)), "k": ParamSpec((k, self.dim)), "v": ParamSpec((v, self.dim)),
                 "o": ParamSpec((self.dim, self.n_heads * self.v_dim))}
        if self.values_are_keys:
            del specs["v"]
        if self.gate:
            specs["g"] = ParamSpec((self.n_heads if self.gate_per_head else self.n_heads * self.v_dim, self.dim))
        if self.qk_norm_weight:
            specs["q_norm"] = ParamSpec((self.head_dim,), role="vector", init="ones_normal")
            specs["k_norm"] = ParamSpec((self.head_dim,), role="vector", init="ones_normal")
        if self.bias:
            specs.update({"q_bias": ParamSpec((q,), role="vector"), "k_bias": ParamSpec((k,), role="vector"),
                          "v_bias": ParamSpec((v,), role="vector")})
        if self.sink:
            specs["sink"] = ParamSpec((self.n_heads,), role="vector")
        return specs

    def bind(self, params):
        if self.gate_per_head and self._tensor_cores(self.runtime.dtype) and torch.device(self.runtime.device).type == "cuda":
            ops.require("latent")                 # the gate per head after the tensor-core kernels (csrc/latent.cu)
        names = ("q", "k") if self.values_are_keys else ("q", "k", "v")
        if self.copy_keys:
            names = ("q", "k", "k")
        self.qkv_width = sum(params[n].shape[0] for n in names)
        # the gate's rows ride in the same product, after q, k and v
        self.wqkv = torch.cat([params[n] for n in names + (("g",) if self.gate else ())], dim=0).contiguous()
        self.wo = params["o"].contiguous()
        if self.bias:
            self.b = torch.cat([params[n + "_bias"].to(torch.float32) for n in names]).contiguous()
        if self.qk_norm_weight:
            self.q_norm = params["q_norm"].contiguous()
            self.k_norm = params["k_norm"].to(self.q_norm.dtype).contiguous()
        if self.sink:
            self.sinks = params["sink"].to(torch.float32).contiguous()
            self.sinks_l2 = ops.sink_table(self.sinks)
        elif self.fixed_sink is not None:
            self.sinks = torch.full((self.n_heads,), self.fixed_sink, dtype=torch.float32, device=self.wo.device)
            self.sinks_l2 = ops.sink_table(self.sinks)

    def _tensor_cores(self, dtype) -> bool:
        return dtype == torch.bfloat16 and self.v_dim == self.head_dim and self.head_dim in (64, 128, 256)

    @property
    def out_width(self) -> int:
        """Width of what ``pre_projection`` returns (the output projection's input)."""
        return self.n_heads * self.v_dim

    def cache_spec(self) -> CacheSpec:
        policy = "chunk" if self.chunk else ("window" if self.window else "full")
        span = self.chunk or self.window or None
        if self.values_are_keys and not self.copy_keys:
            return CacheSpec(policy, (self.n_kv_heads * self.head_dim,), span, tensors=1)
        if self.v_dim == self.head_dim:
            return CacheSpec(policy, (self.n_kv_heads, self.head_dim), span)
        return CacheSpec(policy, (self.n_kv_heads * (self.head_dim + self.v_dim),), span, tensors=1)

    def forward(self, x, ctx, cache):
        out = self.pre_projection(x, ctx, cache)
        with bucket("attn.o_proj"):
            return ops.linear(out, self.wo)

    def pre_projection(self, x, ctx, cache, out=None, out_scale: float = 1.0):
        """The attended (and gated) heads [n, H * v_dim] in the run dtype, times ``out_scale``; written into ``out``
        (a view of the leading columns of wider rows) when given."""
        n = x.shape[0]
        H, G, hd, vd = self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim
        tables = ctx.tables[cache.group]
        pos = self.position
        with bucket("attn.qkv_proj"):
            proj = ops.linear(x, self.wqkv, out_dtype=torch.float32)
        qkv = proj[:, :self.qkv_width]
        gate = proj[:, self.qkv_width:] if self.gate else None
        with bucket("attn.rope"):
            q = ops.qkv_prepare(qkv, H, G, hd, 0 if self.values_are_keys and not self.copy_keys else vd, self.b, getattr(pos, "inv_freq", None),
                                getattr(pos, "rotary_dim", 0), getattr(pos, "interleaved", False),
                                getattr(pos, "magnitude", 1.0), self.qk_norm_eps, ctx.positions, ctx.tok_entry,
                                tables.kv_indptr, tables.kv_indices, cache.kv, tables.page_size, write_kv=cache.owner,
                                q_norm=self.q_norm, k_norm=self.k_norm, norm_first=self.qk_norm_first)
        if out is None:
            out = torch.empty((n, H * vd), dtype=x.dtype, device=x.device)
        with bucket("attn.compute"):
            if self._tensor_cores(x.dtype):
                # bfloat16 heads of 64, 128 or 256 with values as wide as keys: the plain attention part's tensor-core
                # kernels, which take the masks, the sink and the soft cap; gate and factor follow in a kernel of
                # their own
                direct = not self.gate and out_scale == 1.0 and out.is_contiguous()
                heads = out if direct else torch.empty((n, H * vd), dtype=x.dtype, device=x.device)
                ops.paged_attention(q, heads, cache.kv, ctx, tables, H, G, hd, self.scale, self.window, self.chunk,
                                    self.sinks, self.sinks_l2, self.softcap)
                if not direct and self.gate_per_head and out_scale == 1.0 and out.is_contiguous():
                    # one logit per head: the heads [n, H * vd] read as [H, n, vd]
                    ops.gate_heads(heads.view(n, H, vd).transpose(0, 1), gate, out)
                elif not direct:
                    if self.gate_per_head:
                        gate = gate.repeat_interleave(vd, dim=1)
                    ops.gate_mul(heads, gate, out, out_scale)
            else:
                ops.masked_attention(q, out, cache.kv, ctx, tables, H, G, hd, vd, self.scale, self.window, self.chunk,
                                     self.sinks, self.softcap, self.values_are_keys and not self.copy_keys, gate,
                                     out_scale, gate_per_head=self.gate_per_head)
        return out
