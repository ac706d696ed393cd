"""The Finolix design as a model description: pre-norm layers whose norms store their weight around zero (the factor
is 1 + w) and whose branches are multiplied column by column by learned vectors; the residual either one stream or
several that learned coefficients mix (hyper-connections: a sublayer reads a weighted sum of the streams and its
result joins all of them); per layer one of two mixers, latent attention with a sliding window and a sink logit per
head (queries and keys/values through normed latents, one rotated key part shared by the heads, YaRN rotation of
adjacent pairs), or grouped-query causal attention with a weighted RMS norm on every q and k head before a rotation
by halves and a sigmoid gate per head; a feed-forward that is two matrices around a squared relu, routed
silu-gated experts weighted by the softmax over the chosen logits, or absent; layers that run with another layer's
weights and a cache of their own; a final norm and an untied head.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.hc{1,2}.{in, out,
mix}``, ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, o}`` or ``l<i>.mix.{q, k, v, q.norm, k.norm, g,
o}``, ``l<i>.mlp.{up, down}`` or ``l<i>.mlp.{router, router.b, e<j>.gate, e<j>.up, e<j>.down}``, ``final.norm``,
``head``; i counts every listed layer, also those without tensors."""
from __future__ import annotations

from ..config.finolix_config import FinolixConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry


def build_finolix(cfg: FinolixConfig) -> ModelSpec:
    d, S = cfg.width, cfg.streams
    norm = PartSpec("rmsnorm", dict(dim=d, eps=cfg.norm_eps, one_plus=True))
    scale = PartSpec("channel", dict(dim=d))
    hc = PartSpec("hyper_connection", dict(streams=S)) if S else None
    layers, ignore = [], []
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        names = {"norm1.weight": p + "norm1", "scale1.weight": p + "ls1"}
        if layer["type"] == "latent_attention":
            rot = m["rot"]
            scaling = dict(rope_type="yarn", **rot["scaling"]) if rot.get("scaling") else None
            position = PartSpec("rope", dict(head_dim=m["rot_dim"], theta=rot["base"], scaling=scaling,
                                             rotary_dim=rot["dims"], interleaved=True))
            mixer = PartSpec("latent_attention", dict(
                dim=d, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
                q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"], eps=cfg.norm_eps, position=position,
                gated=False, window=(m.get("mask") or {}).get("size") or 0, sink=True))
            names.update({"mixer.dq_norm": p + "mix.dq.norm", "mixer.dkv_norm": p + "mix.dkv.norm"})
            names.update({f"mixer.{k}": p + "mix." + k for k in ("dq", "uq", "dkv", "uk", "uv", "sink", "o")})
        else:
            rot = m.get("rot")
            if rot and rot["dims"]:
                scaling = dict(rope_type="yarn", **rot["scaling"]) if rot.get("scaling") else None
                position = PartSpec("rope", dict(head_dim=m["dim"], theta=rot["base"], scaling=scaling,
                                                 rotary_dim=rot["dims"], interleaved=False))
            else:
                position = PartSpec("none")
            mixer = PartSpec("sink_attention", dict(
                dim=d, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                scale=m["scale"], position=position, qk_norm_eps=cfg.norm_eps, qk_norm_weight=True,
                qk_norm_first=True, gate="head", window=(m.get("mask") or {}).get("size")))
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "g", "o")})
            names.update({"mixer.q_norm": p + "mix.q.norm", "mixer.k_norm": p + "mix.k.norm"})
        parts = {"norm1": norm, "mixer": mixer, "scale1": scale}
        if S:
            parts["hc1"] = hc
            names.update({f"hc1.{k}": f"{p}hc1.{k}" for k in ("in", "out", "mix")})
        f = layer.get("mlp")
        if f is None:
            layers.append(LayerSpec(parts, names, "hyper_prenorm_mixer" if S else "prenorm_mixer_scaled"))
            # a second norm, scale and coefficients without a feed-forward are never applied
            ignore += [p + "norm2", p + "ls2"] + [f"{p}hc2.{k}" for k in ("in", "out", "mix")]
            continue
        names.update({"norm2.weight": p + "norm2", "scale2.weight": p + "ls2"})
        if f["kind"] == "dense":
            ffn = PartSpec("mlp", dict(dim=d, intermediate=f["ff"], activation="relu2"))
            names.update({f"ffn.{k}": p + "mlp." + k for k in ("up", "down")})
        else:
            E = f["router"]["experts"]
            ffn = PartSpec("routed_glu", dict(dim=d, intermediate=f["expert"]["ff"], n_experts=E,
                                              top=f["router"]["top"]))
            names.update({"ffn.router": p + "mlp.router", "ffn.router_bias": p + "mlp.router.b"})
            for e in range(E):
                names.update({f"ffn.{k}{e}": f"{p}mlp.e{e}.{k}" for k in ("gate", "up", "down")})
        parts.update({"norm2": norm, "ffn": ffn, "scale2": scale})
        if S:
            parts["hc2"] = hc
            names.update({f"hc2.{k}": f"{p}hc2.{k}" for k in ("in", "out", "mix")})
        layers.append(LayerSpec(parts, names, "hyper_prenorm" if S else "prenorm_scaled"))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=d, layers=layers, order=[RunEntry(j) for j in cfg.run_order()],
        final_norm=norm, embed_name="embed", final_norm_names={"weight": "final.norm"}, lm_head_name="head",
        ignore_names=tuple(ignore), streams=S)
