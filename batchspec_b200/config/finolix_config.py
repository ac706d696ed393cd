"""Configuration of the Finolix design: a decoder whose ``config.json`` lists its layers one by one; a layer may
borrow another layer's weights; the residual may be kept as several streams.

    {"architecture": "Finolix", "vocab": V, "width": d, "norm": {"eps": e}, "streams": S,
     "layers": [{"type": "latent_attention" | "attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F} | {"kind": "moe", "expert": {"ff": F},
                         "router": {"experts": E, "top": k}} | null,
                 "weights_of": j}, ...]}

A ``latent_attention`` mixer gives heads, dim (unrotated numbers per head), rot_dim, vdim, q_rank, kv_rank, scale,
``rot`` {base, dims, scaling {factor, original, fast, slow} or nothing} and ``mask`` {size}: a sliding window, or
nothing.  An ``attention`` mixer gives heads, kv_heads, dim, vdim, scale, ``rot`` {base, dims} or nothing, and may
give ``mask`` {size} too (a sliding window; without it every earlier position is seen).
``weights_of``: the layer has no tensors of its own and runs with layer j's, with a cache of its own.  ``streams``
absent: one residual stream.  Every size and constant is read from here; keys this reader does not know are listed in
``unread_keys``."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from .model_config import ConfigError, _take, register_config_class

_TOP = {"architecture", "architectures", "vocab", "width", "norm", "streams", "layers"}
_LATENT = {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot", "mask"}
_ATTENTION = {"heads", "kv_heads", "dim", "vdim", "scale", "rot", "mask"}
_SCALING = {"factor", "original", "fast", "slow"}


def _unknown(d: Dict[str, Any], known, where: str, out: List[str]) -> None:
    out.extend(f"{where}{k}" for k in sorted(set(d) - set(known)))


def _positive(d: Dict[str, Any], keys, where: str) -> None:
    for key in keys:
        if _take(d, key, int) <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be positive")


def _rotation(m: Dict[str, Any], where: str, limit: int, unread: List[str]) -> None:
    rot = m.get("rot")
    if rot is None:
        return
    _unknown(rot, {"base", "dims", "scaling"}, where + ".rot.", unread)
    if not _take(rot, "base", float) > 0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive")
    dims = _take(rot, "dims", int)
    if dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}")
    if rot.get("scaling"):
        _unknown(rot["scaling"], _SCALING, where + ".rot.scaling.", unread)
        for key in _SCALING:
            _take(rot["scaling"], key, float)


@dataclass(frozen=True)
class FinolixConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    streams: int                    # 0: one residual stream
    layers: Tuple[Dict[str, Any], ...]
    unread_keys: Tuple[str, ...] = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "FinolixConfig":
        unread: List[str] = []
        _unknown(d, _TOP, "", unread)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = d.get("norm") or {}
        _unknown(norm, {"eps"}, "norm.", unread)
        streams = d.get("streams")
        if streams is not None and not 0 < _take(d, "streams", int) <= 16:
            raise ConfigError("config.json: 'streams' must be between 1 and 16 (or absent)")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _unknown(layer, {"type", "mixer", "mlp", "weights_of"}, where + ".", unread)
            kind, m = layer.get("type"), layer.get("mixer") or {}
            where_m = where + ".mixer"
            if kind == "latent_attention":
                _unknown(m, _LATENT, where_m + ".", unread)
                _positive(m, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"), where_m)
                _take(m, "scale", float)
                if m.get("rot") is None:
                    raise ConfigError(f"config.json: {where_m}.rot is missing (the rotated key part needs it)")
                _rotation(m, where_m, m["rot_dim"], unread)
                if m["rot"]["dims"] != m["rot_dim"]:
                    raise ConfigError(f"config.json: {where_m}.rot.dims must equal rot_dim")
            elif kind == "attention":
                _unknown(m, _ATTENTION, where_m + ".", unread)
                _positive(m, ("heads", "kv_heads", "dim", "vdim"), where_m)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {where_m}.heads must be a multiple of kv_heads")
                _take(m, "scale", float)
                _rotation(m, where_m, m["dim"], unread)
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  f"(known: 'latent_attention', 'attention')")
            mask = m.get("mask")
            if mask is not None:
                _unknown(mask, {"size"}, where_m + ".mask.", unread)
                if _take(mask, "size", int) <= 0:
                    raise ConfigError(f"config.json: {where_m}.mask.size must be positive")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind") == "dense":
                    _unknown(f, {"kind", "ff"}, where + ".mlp.", unread)
                    _positive(f, ("ff",), where + ".mlp")
                elif f.get("kind") == "moe":
                    _unknown(f, {"kind", "expert", "router"}, where + ".mlp.", unread)
                    _unknown(f.get("expert") or {}, {"ff"}, where + ".mlp.expert.", unread)
                    _positive(f.get("expert") or {}, ("ff",), where + ".mlp.expert")
                    r = f.get("router") or {}
                    _unknown(r, {"experts", "top"}, where + ".mlp.router.", unread)
                    _positive(r, ("experts", "top"), where + ".mlp.router")
                    if r["top"] > r["experts"]:
                        raise ConfigError(f"config.json: {where}.mlp.router cannot choose {r['top']} of {r['experts']}")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {f.get('kind')!r} is not known "
                                      f"('dense', 'moe' or null)")
            j = layer.get("weights_of")
            if j is not None:
                if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(layers) or j == i or \
                        layers[j].get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer with tensors of its own")
                if layers[j].get("type") != kind:
                    raise ConfigError(f"config.json: {where} borrows layer {j}'s weights but is of another type")
            out.append(copy.deepcopy(layer))
        cfg = cls(architecture=d.get("architecture") or (d.get("architectures") or [None])[0],
                  vocab_size=_take(d, "vocab", int), width=_take(d, "width", int), norm_eps=_take(norm, "eps", float),
                  streams=int(streams or 0), layers=tuple(out), unread_keys=tuple(unread))
        if cfg.vocab_size <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: vocab and width must be positive and norm.eps > 0")
        return cfg

    def run_order(self) -> List[int]:
        """Per layer run, the index (among the layers that have tensors) of the layer whose weights it uses."""
        own = [i for i, layer in enumerate(self.layers) if layer.get("weights_of") is None]
        return [own.index(layer.get("weights_of", i) if layer.get("weights_of") is not None else i)
                for i, layer in enumerate(self.layers)]

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.streams:
            d["streams"] = self.streams
        return d


register_config_class("Finolix", FinolixConfig)
