"""A plain, slow implementation of the Tokolorn design in float64 on the CPU: whole sequences, one function per
mechanism, python loops where the definition is a recurrence.  It shares no code with the package; the tests compare
the engine with it.

Notation: h is a [T, d] matrix of one sequence's rows, W x means ``x @ W.T`` for a weight stored [out, in]."""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return rms(x, eps) * f64(g).reshape(())


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed_rows(tokens: Sequence[int], table, bigram, scale: float, buckets: int, mul_prev: int, mul_cur: int):
    """embed[token] * scale + bigram[hash(previous token, token)]; the first token takes the table's last row."""
    rows = []
    for i, t in enumerate(tokens):
        r = buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets
        rows.append(f64(table[t]) * scale + f64(bigram[r]))
    return torch.stack(rows)


def decaying_linear_attention(q, k, v, decay: Sequence[float]):
    """q, k [T, H, D], v [T, H, V]: per head S_t = decay_h S_(t-1) + k_t v_t^T (S_0 = 0), o_t = S_t^T q_t."""
    T, heads, dim = q.shape
    out = torch.zeros(T, heads, v.shape[2], dtype=F)
    for j in range(heads):
        S = torch.zeros(dim, v.shape[2], dtype=F)
        for t in range(T):
            S = decay[j] * S + torch.outer(k[t, j], v[t, j])
            out[t, j] = S.T @ q[t, j]
    return out


def lightning(h, w: Dict[str, torch.Tensor], decay: Sequence[float], heads: int, dim: int, vdim: int, eps: float):
    """Linear attention with a fixed decay per head on silu(q), silu(k), silu(v); then the RMS norm over all heads
    together (a weight per coordinate), the sigmoid gate and the output projection."""
    T = h.shape[0]
    q = silu(h @ f64(w["q"]).T).view(T, heads, dim)
    k = silu(h @ f64(w["k"]).T).view(T, heads, dim)
    v = silu(h @ f64(w["v"]).T).view(T, heads, vdim)
    out = decaying_linear_attention(q, k, v, decay)
    o = rms(out.reshape(T, heads * vdim), eps) * f64(w["norm"])
    o = o * torch.sigmoid(h @ f64(w["g"]).T)
    return o @ f64(w["o"]).T


def rotate_interleaved(x, base: float, dims: int):
    """x [T, H, D]: the pairs (2i, 2i+1), i < dims/2, of the token at position p turn by p * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = torch.arange(T, dtype=F) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale: float, visible, softcap: float = 0.0, sink_one: bool = False):
    """q [T, H, D], k [T, G, D], v [T, G, V]; ``visible(i, j)`` says whether query i sees key j <= i.  ``softcap``
    c > 0: s <- c tanh(s / c).  ``sink_one``: the denominator gets one more term exp(0)."""
    T, H, _ = q.shape
    G = k.shape[1]
    see = torch.tensor([[j <= i and bool(visible(i, j)) for j in range(T)] for i in range(T)])
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        e = torch.where(see, torch.exp(s), torch.zeros((), dtype=F))
        p = e / (e.sum(dim=1, keepdim=True) + (1.0 if sink_one else 0.0))
        out[:, hh] = p @ v[:, g]
    return out


def window_attention(h, w, m: dict):
    """Grouped-query attention with rotary positions, a soft cap on the scores, a sliding window and an output gate."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ f64(w["q"]).T).view(T, H, D)
    k = (h @ f64(w["k"]).T).view(T, G, D)
    v = (h @ f64(w["v"]).T).view(T, G, V)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q, k = rotate_interleaved(q, rot["base"], rot["dims"]), rotate_interleaved(k, rot["base"], rot["dims"])
    size = (m.get("mask") or {}).get("size")
    visible = (lambda i, j: i - j < size) if size else (lambda i, j: True)
    o = softmax_attention(q, k, v, m["scale"], visible, softcap=m.get("softcap") or 0.0).reshape(T, H * V)
    o = o * torch.sigmoid(h @ f64(w["g"]).T)
    return o @ f64(w["o"]).T


def causal_conv(x, conv, bias):
    """x [T, C], conv [C, taps], bias [C]: y_t = bias + sum_j conv[:, j] x_(t - (taps-1) + j), zeros before the start
    (the last column multiplies the token's own input)."""
    T, taps = x.shape[0], conv.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        acc = bias.clone()
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                acc = acc + conv[:, j] * x[src]
        y[t] = acc
    return y


def softplus(x):
    return torch.where(x > 40, x, torch.log1p(torch.exp(torch.clamp(x, max=40))))


def diagonal_scan(x, dt, A, B, C, D):
    """x, dt [T, I], A [I, N], B, C [T, N], D [I]: S <- exp(dt A) S + dt x B^T per channel, y = S C + D x."""
    T, inner = x.shape
    S = torch.zeros(inner, A.shape[1], dtype=F)
    y = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = (S * C[t][None, :]).sum(1) + D * x[t]
    return y


def selective_scan(h, w, m: dict):
    """Mamba: in-projection [x | z], causal convolution and silu on x, input-dependent step dt, B and C, a diagonal
    state per channel, a skip D x, the gate silu(z) and the output projection."""
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ f64(w["in"]).T
    x, z = xz[:, :inner], xz[:, inner:]
    xc = silu(causal_conv(x, f64(w["conv"]), f64(w["conv.b"])))
    p = xc @ f64(w["x"]).T
    dt, B, C = p[:, :R], p[:, R:R + N], p[:, R + N:R + 2 * N]
    dt = softplus(dt @ f64(w["dt"]).T + f64(w["dt.b"]))
    y = diagonal_scan(xc, dt, -torch.exp(f64(w["A_log"])), B, C, f64(w["D"]))
    return (y * silu(z)) @ f64(w["o"]).T


def parallel_mixer(h, w, m: dict):
    left = window_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"])
    right = selective_scan(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def chunk_attention(h, w, m: dict):
    """Grouped-query attention whose values are its keys, without positions, over the keys of the query's own chunk,
    with one added to the softmax's denominator."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ f64(w["q"]).T).view(T, H, D)
    k = (h @ f64(w["k"]).T).view(T, G, D)
    size = (m.get("mask") or {}).get("size")
    visible = (lambda i, j: i // size == j // size) if size else (lambda i, j: True)
    o = softmax_attention(q, k, k, m["scale"], visible, sink_one=True).reshape(T, H * D)
    return o @ f64(w["o"]).T


def feed_forward(h, w):
    return (gelu_tanh(h @ f64(w["gate"]).T) * (h @ f64(w["up"]).T)) @ f64(w["down"]).T


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {}
    a, b, times = loop.get("start", 0), loop.get("stop", 0), loop.get("times", 1)
    if b <= a or times <= 1:
        return list(range(n))
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def layer_forward(x, cfg: dict, tensors: Dict[str, torch.Tensor], i: int):
    layer, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    w = {k[len(p) + 4:]: v for k, v in tensors.items() if k.startswith(p + "mix.")}
    h = scalar_norm(x, tensors[p + "norm1"], eps)
    m = layer["mixer"]
    if layer["type"] == "lightning":
        y = lightning(h, w, m["decay"], m["heads"], m["dim"], m["vdim"], eps)
    elif layer["type"] == "parallel":
        y = parallel_mixer(h, w, m)
    elif layer["type"] == "attention":
        y = chunk_attention(h, w, m)
    else:
        raise ValueError(layer["type"])
    x = x + y * f64(tensors[p + "ls1"])
    if layer.get("mlp") is not None:
        fw = {k[len(p) + 4:]: v for k, v in tensors.items() if k.startswith(p + "mlp.")}
        x = x + feed_forward(scalar_norm(x, tensors[p + "norm2"], eps), fw) * f64(tensors[p + "ls2"])
    return x


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """float64 logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    e = cfg["embedding"]
    bg = e.get("bigram")
    x = f64(tensors["embed"])[list(tokens)] * e.get("scale", 1.0)
    if bg:
        x = embed_rows(tokens, tensors["embed"], tensors["bigram"], e.get("scale", 1.0), bg["buckets"], bg["mul_prev"],
                       bg["mul_cur"])
    after = []
    for i in run_order(cfg):
        x = layer_forward(x, cfg, tensors, i)
        after.append(x.clone())
    z = scalar_norm(x, tensors["final.norm"], cfg["norm"]["eps"])
    logits = (z @ f64(tensors["head"]).T) * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(after)) if return_layers else logits


# ---------------------------------------------------------------------------------------------- a model folder
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
            arr = np.frombuffer(data[lo:hi], dtype={"F32": np.float32, "I32": np.int32, "F64": np.float64}[meta["dtype"]]).copy()
        out[name] = torch.from_numpy(arr.copy()).reshape(meta["shape"])
    return out


def read_model_folder(folder):
    import json
    from pathlib import Path
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_tensors(folder / "model.safetensors")
