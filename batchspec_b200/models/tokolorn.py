"""The Tokolorn design as a model description: the embedding times a constant plus a row of a hashed bigram table;
pre-norm layers whose norms have one number as weight and whose branches are multiplied column by column by learned
vectors before the residual sum; per layer one of three mixers, lightning attention (a decaying [key x value] state
per head), a sliding-window attention with a soft cap and an output gate side by side with a selective scan, or a
chunk-masked attention whose values are its keys and whose softmax has one added to the denominator; a gelu-gated
feed-forward or none; a span of layers that runs several times in a row with shared weights and separate caches and
state; a final norm, an untied head and a constant on the logits.

Checkpoint names: ``embed``, ``bigram``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``,
``l<i>.mix.{q, k, v, g, o, norm}``, ``l<i>.mix.left.{q, k, v, g, o}``,
``l<i>.mix.right.{in, conv, conv.b, x, dt, dt.b, A_log, D, o}``, ``l<i>.mlp.{gate, up, down}``, ``final.norm``,
``head``."""
from __future__ import annotations

from ..config.tokolorn_config import TokolornConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

_RIGHT_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b",
                "A_log": "A_log", "D": "D", "o": "o"}


def build_tokolorn(cfg: TokolornConfig) -> ModelSpec:
    d = cfg.width
    norm = PartSpec("rmsnorm", dict(dim=d, eps=cfg.norm_eps, single_rounding=True, scalar_weight=True))
    scale = PartSpec("channel", dict(dim=d))
    layers, ignore = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        names = {"norm1.weight": p + "norm1", "scale1.weight": p + "ls1"}
        if layer["type"] == "lightning":
            mixer = PartSpec("lightning_attention", dict(dim=d, n_heads=m["heads"], head_dim=m["dim"], v_dim=m["vdim"],
                                                         decay=list(m["decay"]), eps=cfg.norm_eps))
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "g", "norm", "o")})
        elif layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            rot = a.get("rot")
            position = (PartSpec("rope", dict(head_dim=a["dim"], theta=rot["base"], scaling=None, rotary_dim=rot["dims"],
                                              interleaved=True)) if rot and rot["dims"] else PartSpec("none"))
            left = PartSpec("sink_attention", dict(
                dim=d, n_heads=a["heads"], n_kv_heads=a["kv_heads"], head_dim=a["dim"], v_dim=a["vdim"],
                scale=a["scale"], position=position, window=(a.get("mask") or {}).get("size"),
                softcap=a.get("softcap"), gate=True))
            right = PartSpec("selective_scan", dict(dim=d, inner=b["inner"], n_state=b["state"], dt_rank=b["dt_rank"],
                                                    taps=b["conv"]))
            mixer = PartSpec("parallel", dict(left=left, right=right, left_scale=m["left_scale"],
                                              right_scale=m["right_scale"]))
            names.update({f"mixer.left.{k}": p + "mix.left." + k for k in ("q", "k", "v", "g", "o")})
            names.update({f"mixer.right.{k}": p + "mix.right." + v for k, v in _RIGHT_NAMES.items()})
        else:
            mixer = PartSpec("sink_attention", dict(
                dim=d, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                scale=m["scale"], position=PartSpec("none"), chunk=(m.get("mask") or {}).get("size"),
                fixed_sink=0.0, values_are_keys=True))
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "o")})
        f = layer.get("mlp")
        if f is None:
            layers.append(LayerSpec({"norm1": norm, "mixer": mixer, "scale1": scale}, names, "prenorm_mixer_scaled"))
            ignore += [p + "norm2", p + "ls2"]           # a second norm and scale without a feed-forward are never applied
            continue
        names.update({"norm2.weight": p + "norm2", "scale2.weight": p + "ls2"})
        names.update({f"ffn.{k}": p + "mlp." + k for k in ("gate", "up", "down")})
        ffn = PartSpec("swiglu", dict(dim=d, intermediate=f["ff"], activation="gelu_tanh"))
        layers.append(LayerSpec({"norm1": norm, "mixer": mixer, "scale1": scale, "norm2": norm, "ffn": ffn,
                                 "scale2": scale}, names, "prenorm_scaled"))
    spec = ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=d, layers=layers, order=[RunEntry(i) for i in cfg.run_order()],
        final_norm=norm, embed_name="embed", final_norm_names={"weight": "final.norm"}, lm_head_name="head",
        ignore_names=tuple(ignore), embed_scale=cfg.embed_scale)
    if cfg.bigram is not None:
        spec.input_part = PartSpec("bigram_hash", dict(dim=d, vocab=cfg.vocab_size, **cfg.bigram))
        spec.input_names = {"table": "bigram"}
    if cfg.logit_scale != 1.0:
        spec.logits_part = PartSpec("scale", dict(factor=cfg.logit_scale))
    return spec
