"""A plain, slow implementation of the Finolix design in float64 on the CPU: whole sequences, one function per
mechanism.  It shares no code with the package; the tests compare the engine with it.

Notation: h is a [T, d] matrix of one sequence's rows, W x means ``x @ W.T`` for a weight stored [out, in]."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms(x, eps) * (1.0 + f64(w))


def weighted_norm(x, w, eps):
    return rms(x, eps) * f64(w)


def silu(z):
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------- rotation

def yarn_frequencies(base: float, dims: int, scaling: Optional[dict]):
    """f_i = base^(-2i/dims); with YaRN blended towards f_i / factor along a ramp over the pair index.  Returns the
    frequencies and the factor on cosine and sine."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions: Sequence[int], freqs: Sequence[float], magnitude: float, interleaved: bool):
    """x [T, H, D]: pair i of the first 2 * len(freqs) numbers of a head turns by position * freqs[i]; the pair is
    (2i, 2i + 1) when interleaved, else (i, i + len(freqs))."""
    out = x.clone()
    half = len(freqs)
    p = torch.tensor(list(positions), dtype=F)
    for i, f in enumerate(freqs):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        c, s = (torch.cos(p * f) * magnitude)[:, None], (torch.sin(p * f) * magnitude)[:, None]
        u, v = x[:, :, a], x[:, :, b]
        out[:, :, a] = u * c - v * s
        out[:, :, b] = v * c + u * s
    return out


# ---------------------------------------------------------------------------- attention

def softmax_attention(q, k, v, scale: float, window: Optional[int] = None, sink=None):
    """q [T, H, D], k [T, H, D], v [T, H, V] (one key/value head per query head already).  Token i sees j <= i and,
    with a window, i - j < window.  ``sink`` [H]: exp(sink_h) joins the denominator."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e[:, None] * v[lo:i + 1, h]).sum(0) / den
    return out


def latent_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, positions=None):
    """Queries through a normed latent; keys and values from one normed latent per token plus one rotated key part
    shared by the heads; a sliding window and a sink logit per head."""
    T = h.shape[0]
    H, D, P, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = list(range(T)) if positions is None else positions
    cq = weighted_norm(h @ f64(w["dq"]).T, w["dq.norm"], eps)
    q = (cq @ f64(w["uq"]).T).view(T, H, D + P)
    down = h @ f64(w["dkv"]).T
    c = weighted_norm(down[:, :R], w["dkv.norm"], eps)
    kr = down[:, R:].view(T, 1, P)
    k_plain = (c @ f64(w["uk"]).T).view(T, H, D)
    v = (c @ f64(w["uv"]).T).view(T, H, V)
    rot = m["rot"]
    freqs, mag = yarn_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
    q_rot = rotate(q[:, :, D:], positions, freqs, mag, True)
    k_rot = rotate(kr, positions, freqs, mag, True).expand(T, H, P)
    qq = torch.cat([q[:, :, :D], q_rot], dim=2)
    kk = torch.cat([k_plain, k_rot], dim=2)
    window = (m.get("mask") or {}).get("size")
    out = softmax_attention(qq, kk, v, m["scale"], window, f64(w["sink"]))
    return out.reshape(T, H * V) @ f64(w["o"]).T


def gated_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, positions=None):
    """Grouped-query causal attention: a weighted RMS norm on every q and k head before the rotation of the head's
    first numbers by halves, an ordinary softmax, a sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T)) if positions is None else positions
    q = weighted_norm((h @ f64(w["q"]).T).view(T, H, D), w["q.norm"], eps)
    k = weighted_norm((h @ f64(w["k"]).T).view(T, G, D), w["k.norm"], eps)
    v = (h @ f64(w["v"]).T).view(T, G, V)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        freqs, mag = yarn_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q, k = rotate(q, positions, freqs, mag, False), rotate(k, positions, freqs, mag, False)
    per = H // G
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    out = softmax_attention(q, k, v, m["scale"])
    out = out * torch.sigmoid(h @ f64(w["g"]).T)[:, :, None]
    return out.reshape(T, H * V) @ f64(w["o"]).T


# ---------------------------------------------------------------------------- feed-forwards

def squared_relu_mlp(h, w):
    return (torch.relu(h @ f64(w["up"]).T) ** 2) @ f64(w["down"]).T


def route(h, router, bias, top: int):
    """Per token the ``top`` experts of largest logit and the softmax over those logits alone."""
    z = h @ f64(router).T + f64(bias)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def routed_experts(h, w, n_experts: int, top: int):
    idx, wt = route(h, w["router"], w["router.b"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            g, u, d = f64(w[f"e{e}.gate"]), f64(w[f"e{e}.up"]), f64(w[f"e{e}.down"])
            out[t] += wt[t, j] * ((silu(g @ h[t]) * (u @ h[t])) @ d.T)
    return out


# ---------------------------------------------------------------------------- the model

def _sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], round_input=None):
    """Logits [T, vocab] and the residual stream after every layer run [runs, T, width] (the sum of the streams
    when there are several).  ``round_input``: applied to every sublayer's input (None: nothing)."""
    eps = config["norm"]["eps"]
    x = f64(tensors["embed"])[list(tokens)]
    s = config.get("streams")
    xs = [x.clone() for _ in range(s)] if s else None
    after = []
    rnd = round_input or (lambda t: t)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i if layer.get('weights_of') is None else layer['weights_of']}."
        subs = [(1, "mix.", lambda u, w: (latent_attention if layer["type"] == "latent_attention" else gated_attention)(
            u, w, layer["mixer"], eps))]
        f = layer.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                subs.append((2, "mlp.", lambda u, w: squared_relu_mlp(u, w)))
            else:
                subs.append((2, "mlp.", lambda u, w, f=f: routed_experts(u, w, f["router"]["experts"], f["router"]["top"])))
        for q, prefix, fn in subs:
            norm_w, ls = tensors[f"{p}norm{q}"], f64(tensors[f"{p}ls{q}"])
            if xs is None:
                x = x + ls * fn(rnd(one_plus_norm(x, norm_w, eps)), _sub(tensors, p + prefix))
                continue
            a, b, mix = (f64(tensors[f"{p}hc{q}.{n}"]) for n in ("in", "out", "mix"))
            u = sum(a[j] * xs[j] for j in range(s))
            y = ls * fn(rnd(one_plus_norm(u, norm_w, eps)), _sub(tensors, p + prefix))
            xs = [sum(mix[j, t] * xs[j] for j in range(s)) + b[t] * y for t in range(s)]
        after.append(x.clone() if xs is None else sum(xs))
    x = x if xs is None else sum(xs)
    logits = one_plus_norm(x, tensors["final.norm"], eps) @ f64(tensors["head"]).T
    return logits, torch.stack(after)


# ---------------------------------------------------------------------------- model folders

def read_tensors(path) -> Dict[str, torch.Tensor]:
    """A safetensors file: an 8-byte little-endian length, that many bytes of JSON (name -> dtype, shape, offsets), the
    data.  bfloat16 comes back as float32 with the same values."""
    import json
    import struct
    import numpy as np
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    data = raw[8 + n:]
    out = {}
    for name, meta in json.loads(raw[8:8 + n]).items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        if meta["dtype"] == "BF16":
            arr = (np.frombuffer(data[lo:hi], dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            arr = np.frombuffer(data[lo:hi], dtype={"F32": np.float32, "I32": np.int32}[meta["dtype"]]).copy()
        out[name] = torch.from_numpy(arr.copy()).reshape(meta["shape"])
    return out


def read_model_folder(folder):
    import json
    from pathlib import Path
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_tensors(folder / "model.safetensors")
