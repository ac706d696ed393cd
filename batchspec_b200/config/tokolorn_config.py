"""Configuration of the Tokolorn design: a decoder whose ``config.json`` lists its layers one by one, some of which may
run several times in a row.

    {"architecture": "Tokolorn", "vocab": V, "width": d, "norm": {"eps": e}, "logit_scale": s,
     "embedding": {"scale": m, "bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "lightning" | "parallel" | "attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

A ``lightning`` mixer gives heads, dim, vdim and decay (a factor per head).  A ``parallel`` mixer gives ``left``
(heads, kv_heads, dim, vdim, scale, softcap, ``mask`` {size}: a sliding window, ``rot`` {base, dims}), ``right``
(inner, state, dt_rank, conv) and left_scale / right_scale.  An ``attention`` mixer gives heads, kv_heads, dim, vdim,
scale and ``mask`` {size}: chunks of that many positions.  ``loop``: layers a .. b-1 run n times in a row with the
same weights.  Every size and constant is read from here; keys this reader does not know are listed in
``unread_keys``."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .model_config import ConfigError, _take, register_config_class

_TOP = {"architecture", "architectures", "vocab", "width", "norm", "logit_scale", "embedding", "layers", "loop"}
_LIGHTNING = {"heads", "dim", "vdim", "decay"}
_LEFT = {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask", "rot"}
_RIGHT = {"inner", "state", "dt_rank", "conv"}
_ATTENTION = {"heads", "kv_heads", "dim", "vdim", "scale", "mask"}


def _unknown(d: Dict[str, Any], known, where: str, out: List[str]) -> None:
    out.extend(f"{where}{k}" for k in sorted(set(d) - set(known)))


def _positive(d: Dict[str, Any], keys, where: str) -> None:
    for key in keys:
        if _take(d, key, int) <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be positive")


def _mask(m: Dict[str, Any], where: str, unread: List[str]) -> None:
    mask = m.get("mask")
    if mask is not None:
        _unknown(mask, {"size"}, where + ".mask.", unread)
        if _take(mask, "size", int) <= 0:
            raise ConfigError(f"config.json: {where}.mask.size must be positive")


def _grouped_heads(m: Dict[str, Any], where: str) -> None:
    _positive(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
    _take(m, "scale", float)


@dataclass(frozen=True)
class TokolornConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    logit_scale: float
    embed_scale: float
    bigram: Optional[Dict[str, int]]
    layers: Tuple[Dict[str, Any], ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    unread_keys: Tuple[str, ...] = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "TokolornConfig":
        unread: List[str] = []
        _unknown(d, _TOP, "", unread)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = d.get("norm") or {}
        _unknown(norm, {"eps"}, "norm.", unread)
        emb = d.get("embedding") or {}
        _unknown(emb, {"scale", "bigram"}, "embedding.", unread)
        bigram = emb.get("bigram")
        if bigram is not None:
            _unknown(bigram, {"buckets", "mul_prev", "mul_cur"}, "embedding.bigram.", unread)
            bigram = {k: _take(bigram, k, int) for k in ("buckets", "mul_prev", "mul_cur")}
            if bigram["buckets"] <= 0 or bigram["mul_prev"] < 0 or bigram["mul_cur"] < 0:
                raise ConfigError("config.json: embedding.bigram needs buckets > 0 and multipliers >= 0")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _unknown(layer, {"type", "mixer", "mlp"}, where + ".", unread)
            kind, m = layer.get("type"), layer.get("mixer") or {}
            where_m = where + ".mixer"
            if kind == "lightning":
                _unknown(m, _LIGHTNING, where_m + ".", unread)
                _positive(m, ("heads", "dim", "vdim"), where_m)
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != m["heads"] or \
                        not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    raise ConfigError(f"config.json: {where_m}.decay must list one number per head")
            elif kind == "parallel":
                _unknown(m, {"left", "right", "left_scale", "right_scale"}, where_m + ".", unread)
                left, right = m.get("left") or {}, m.get("right") or {}
                _unknown(left, _LEFT, where_m + ".left.", unread)
                _unknown(right, _RIGHT, where_m + ".right.", unread)
                _grouped_heads(left, where_m + ".left")
                _mask(left, where_m + ".left", unread)
                if left.get("softcap") is not None and not _take(left, "softcap", float) > 0:
                    raise ConfigError(f"config.json: {where_m}.left.softcap must be positive")
                rot = left.get("rot")
                if rot is not None:
                    _unknown(rot, {"base", "dims"}, where_m + ".left.rot.", unread)
                    _take(rot, "base", float)
                    dims = _take(rot, "dims", int)
                    if dims < 0 or dims % 2 or dims > left["dim"]:
                        raise ConfigError(f"config.json: {where_m}.left.rot.dims must be even and at most dim")
                _positive(right, ("inner", "state", "dt_rank", "conv"), where_m + ".right")
                _take(m, "left_scale", float)
                _take(m, "right_scale", float)
            elif kind == "attention":
                _unknown(m, _ATTENTION, where_m + ".", unread)
                _grouped_heads(m, where_m)
                _mask(m, where_m, unread)
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"config.json: {where_m}: the values of this mixer are its keys, so vdim must "
                                      f"equal dim ({m['vdim']} != {m['dim']})")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  f"(known: 'lightning', 'parallel', 'attention')")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {f.get('kind')!r} is not known ('dense' or null)")
                _unknown(f, {"kind", "ff"}, where + ".mlp.", unread)
                if _take(f, "ff", int) <= 0:
                    raise ConfigError(f"config.json: {where}.mlp.ff must be positive")
            out.append(copy.deepcopy(layer))
        loop = d.get("loop") or {}
        _unknown(loop, {"start", "stop", "times"}, "loop.", unread)
        start, stop, times = _take(loop, "start", int, 0), _take(loop, "stop", int, 0), _take(loop, "times", int, 1)
        if not (0 <= start <= stop <= len(out)) or times < 1:
            raise ConfigError(f"config.json: loop {loop} does not fit {len(out)} layers")
        cfg = cls(architecture=d.get("architecture") or (d.get("architectures") or [None])[0],
                  vocab_size=_take(d, "vocab", int), width=_take(d, "width", int), norm_eps=_take(norm, "eps", float),
                  logit_scale=_take(d, "logit_scale", float, 1.0), embed_scale=_take(emb, "scale", float, 1.0),
                  bigram=bigram, layers=tuple(out), loop_start=start, loop_stop=stop, loop_times=times,
                  unread_keys=tuple(unread))
        if cfg.vocab_size <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: vocab and width must be positive and norm.eps > 0")
        return cfg

    def run_order(self) -> List[int]:
        """The layer of every layer run: the layers before the loop, the looped layers ``loop_times`` times in a row,
        the layers after it."""
        n, a, b, times = len(self.layers), self.loop_start, self.loop_stop, self.loop_times
        if b <= a or times <= 1:
            return list(range(n))
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def to_json_dict(self) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": self.embed_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(self.bigram)
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "embedding": emb,
                "layers": copy.deepcopy(list(self.layers)),
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}


register_config_class("Tokolorn", TokolornConfig)
