"""Latent attention: queries and keys/values go through low-rank latents, and the cache keeps one entry per token.

With h a token's normed input, H heads, per head ``dim`` unrotated and ``rot_dim`` rotated query/key numbers,
``vdim`` value numbers, latents of ``q_rank`` and ``kv_rank``:

    cq = RMS(Wdq h) * nq                      q = Wuq cq          per head [dim unrotated | rot_dim rotated]
    [c' | kr] = Wdkv h                        c = RMS(c') * nkv   kr: one rotated key part for all heads
    k_h = Wuk_h c,  v_h = Wuv_h c             score_h(i, j) = (q_h . k_h(j) + rot(qr_h, i) . rot(kr, j)) * scale
    out = Wo concat_h(sigmoid(Wg h)_h * sum_j softmax_j(score_h(i, .)) v_h(j))

Options: ``gated`` False leaves the gate out; ``window`` W keeps the keys i - W + 1 .. i of query i (pages that the
window has passed are given back); ``sink``: a learned logit per head that only enlarges the softmax's denominator
(nothing is attended through it, and ``scale`` does not touch it).

Only [c | rot(kr)] is cached (one tensor per token, ``kv_rank + rot_dim`` numbers).  The per-head keys and values
are never formed: since q_h . (Wuk_h c) = (Wuk_h^T q_h) . c, the unrotated query is taken into the latent space
(one small product per head), attention runs there for all heads over the same entries, and the head's value
up-projection is applied to its attended latent afterwards.  The step's launch sequence:

    one product for [Wdq; Wdkv; Wg] (float32 out) -> latent_prepare (both RMS norms in float32, rotation of kr,
    cache append) -> Wuq -> per-head Wuk^T -> latent attention (which rotates the queries' rotated parts as it
    loads them) -> per-head Wuv -> gate and regroup -> Wo
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import MIXERS, POSITION_ENCODINGS, CacheSpec, Mixer, ParamSpec, PartSpec, Runtime, build_part, register_part


@register_part(MIXERS, "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, n_heads: int, head_dim: int, rot_dim: int, v_dim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, position: PartSpec, gated: bool = True, window: int = 0,
                 sink: bool = False):
        self.runtime = runtime
        self.dim, self.n_heads, self.head_dim, self.rot_dim = int(dim), int(n_heads), int(head_dim), int(rot_dim)
        self.v_dim, self.q_rank, self.kv_rank = int(v_dim), int(q_rank), int(kv_rank)
        self.scale, self.eps, self.gated = float(scale), float(eps), bool(gated)
        self.window, self.sink = int(window or 0), bool(sink)
        if self.window < 0:
            raise ValueError(f"a sliding window is positive, got {window}")
        self.sinks = None
        if self.rot_dim % 2 or self.rot_dim <= 0:
            raise ValueError(f"the rotated part of a head must have an even, positive size, got {rot_dim}")
        if min(self.n_heads, self.head_dim, self.v_dim, self.q_rank, self.kv_rank) <= 0:
            raise ValueError("latent attention needs positive head count, head sizes and ranks")
        self.position = build_part(POSITION_ENCODINGS, position, runtime)
        if getattr(self.position, "rotary_dim", None) != self.rot_dim or not getattr(self.position, "interleaved", False):
            raise ValueError("latent attention rotates adjacent pairs over the whole rotated part")

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, qk = self.n_heads, self.head_dim + self.rot_dim
        specs = {"dq": ParamSpec((self.q_rank, self.dim)),
                 "dq_norm": ParamSpec((self.q_rank,), role="vector", init="ones_normal"),
                 "uq": ParamSpec((H * qk, self.q_rank)),
                 "dkv": ParamSpec((self.kv_rank + self.rot_dim, self.dim)),
                 "dkv_norm": ParamSpec((self.kv_rank,), role="vector", init="ones_normal"),
                 "uk": ParamSpec((H * self.head_dim, self.kv_rank)),
                 "uv": ParamSpec((H * self.v_dim, self.kv_rank)),
                 "o": ParamSpec((self.dim, H * self.v_dim))}
        if self.gated:
            specs["g"] = ParamSpec((H, self.dim))
        if self.sink:
            specs["sink"] = ParamSpec((H,), role="vector")
        return specs

    def bind(self, params):
        if torch.device(self.runtime.device).type == "cuda":
            ops.require("latent")                 # the kernels of csrc/latent*.cu
        H = self.n_heads
        rows = [params["dq"], params["dkv"]] + ([params["g"]] if self.gated else [])
        self.w_down = torch.cat(rows, dim=0).contiguous()                  # [q_rank + kv_rank + rot_dim (+ H), dim]
        self.w_uq = params["uq"].contiguous()
        # Wuk_h^T as the [N, K] operand of "x @ w^T": [H, kv_rank, head_dim]
        self.w_uk_t = params["uk"].view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = params["uv"].view(H, self.v_dim, self.kv_rank).contiguous()
        self.w_o = params["o"].contiguous()
        self.n_q, self.n_kv = params["dq_norm"], params["dkv_norm"]
        if self.n_kv.dtype != self.n_q.dtype:
            self.n_kv = self.n_kv.to(self.n_q.dtype)
        if self.sink:
            self.sinks = params["sink"].to(torch.float32).contiguous()
        if not self.gated:
            self.open_gate = torch.full((1, H), 1e4, dtype=torch.float32, device=self.w_o.device)   # sigmoid -> 1

    def cache_spec(self) -> CacheSpec:
        if self.window:
            return CacheSpec("window", (self.kv_rank + self.rot_dim,), self.window, tensors=1)
        return CacheSpec("full", (self.kv_rank + self.rot_dim,), tensors=1)

    def forward(self, x, ctx, cache):
        n = x.shape[0]
        H, dh, P, R = self.n_heads, self.head_dim, self.rot_dim, self.kv_rank
        tables = ctx.tables[cache.group]
        pos = self.position
        with bucket("attn.down_proj"):
            down = ops.linear(x, self.w_down, out_dtype=torch.float32)
        with bucket("attn.latent_prepare"):
            cq = ops.latent_prepare(down, 0, self.q_rank, self.q_rank, R, P, self.n_q, self.n_kv, self.eps,
                                    pos.inv_freq, pos.magnitude, ctx.positions, ctx.tok_entry, tables.kv_indptr,
                                    tables.kv_indices, cache.kv, tables.page_size, write_kv=cache.owner)
        with bucket("attn.q_proj"):
            q = ops.linear(cq, self.w_uq).view(n, H, dh + P)
        q_rot = q[:, :, dh:]                      # rotated on its way into the attention kernel
        with bucket("attn.absorb"):
            q_lat = ops.linear_batched(q[:, :, :dh].transpose(0, 1), self.w_uk_t)          # [H, n, R]
        o_lat = torch.empty((H, n, R), dtype=x.dtype, device=x.device)
        with bucket("attn.compute"):
            ops.latent_attention(q_lat, q_rot, o_lat, cache.kv, ctx, tables, H, R, P, self.scale,
                                 rotate=(pos.inv_freq, pos.magnitude), window=self.window, sink=self.sinks)
        with bucket("attn.v_proj"):
            v = ops.linear_batched(o_lat, self.w_uv)                                        # [H, n, v_dim]
        heads = torch.empty((n, H * self.v_dim), dtype=x.dtype, device=x.device)
        with bucket("attn.gate"):
            if self.gated:
                gate = down[:, self.q_rank + R + P:self.q_rank + R + P + H]
            else:
                gate = self.open_gate.expand(n, H)                  # every row reads the same logits (row stride 0)
            ops.gate_heads(v, gate, heads)
        with bucket("attn.o_proj"):
            return ops.linear(heads, self.w_o)
