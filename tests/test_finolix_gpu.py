"""The Finolix design on the engine against the plain implementation in ``plain_finolix.py``: every mechanism alone
(kernels against one plain function each), then whole models of configurations that share no size, fed whole, with a
decoded tail, in portions down to two tokens, token by token, in mixed batches over pools that force pages to be used
again, through ``bin/trace_run`` and through the scheduler."""
from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers as H
import plain_finolix as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
F64 = torch.float64


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, window=None, scaling=None, mlp=None, **more):
    rot = dict(base=base, dims=rot_dim)
    if scaling:
        rot["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale, rot=rot)
    if window:
        m["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=m, mlp=mlp, **more)


def _attn(heads, kv_heads, dim, vdim, scale, rot_dims=None, base=None, mlp=None, **more):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if rot_dims is not None:
        m["rot"] = dict(base=base, dims=rot_dims)
    return dict(type="attention", mixer=m, mlp=mlp, **more)


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def _config(vocab, width, eps, layers, streams=None):
    cfg = dict(architecture="Finolix", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if streams:
        cfg["streams"] = streams
    return cfg


def _borrow(layers, j):
    return dict(layers[j], weights_of=j)


# Configurations that share no size.  A: three streams, a window that is no multiple of the page, a layer without a
# feed-forward, a layer run twice more with borrowed weights, rotation of a part of the head.  B: ONE residual stream
# (no coefficients at all), odd sizes (width 100, heads of 6, one expert of which one is taken, no rotation in the
# attention layer, no window in the latent layer).  C: two streams, sizes at which the tensor-core kernels and the
# products' 8-wide loads run in bfloat16 (heads of 64, latents that are multiples of 32).  D: streams = 1 with
# coefficients, grouped heads of unequal key and value size.
_A = [_latent(3, 8, 4, 12, 20, 24, 0.3, 5000.0, window=10, scaling=(4.0, 32, 8.0, 1.0), mlp=_dense(40)),
      _attn(4, 2, 12, 20, 0.25, rot_dims=8, base=3000.0, mlp=_moe(16, 5, 2)),
      _latent(2, 6, 2, 5, 12, 16, 0.4, 100.0, window=7)]
CFG_A = _config(200, 48, 1e-5, _A + [_borrow(_A, 1), _borrow(_A, 0), _borrow(_A, 1)], streams=3)
CFG_B = _config(513, 100, 1e-6, [_attn(2, 1, 6, 6, 0.4, mlp=_moe(36, 1, 1)),
                                 _latent(5, 10, 6, 7, 30, 40, 0.2, 1e6, mlp=_moe(20, 7, 7)),
                                 _attn(3, 3, 10, 4, 0.3, rot_dims=10, base=20.0, mlp=_dense(44))])
_C = [_latent(8, 32, 32, 48, 96, 128, 0.125, 1e6, window=80, scaling=(2.0, 64, 32.0, 1.0), mlp=_moe(64, 8, 2)),
      _attn(8, 2, 64, 64, 0.125, rot_dims=32, base=250000.0, mlp=_dense(192)),
      _latent(4, 64, 16, 64, 64, 64, 0.1, 10000.0, mlp=_moe(96, 6, 3))]
CFG_C = _config(640, 320, 1e-5, _C + [_borrow(_C, 0)], streams=2)
CFG_D = _config(90, 40, 1e-5, [_attn(6, 3, 8, 12, 0.35, rot_dims=8, base=1000.0, mlp=_dense(24)),
                               _latent(1, 16, 8, 24, 8, 8, 0.2, 50.0, window=1, mlp=_dense(32))], streams=1)
# one latent layer with a window of 12 and four streams: a changed token reaches other positions through it alone
CFG_WINDOW = _config(150, 32, 1e-5, [_latent(2, 8, 8, 8, 16, 16, 0.5, 1000.0, window=12, mlp=_dense(24))], streams=4)
CONFIGS = {"A": (CFG_A, 11, 4), "B": (CFG_B, 12, 8), "C": (CFG_C, 13, 16), "D": (CFG_D, 14, 4),
           "WINDOW": (CFG_WINDOW, 15, 8)}
LENGTHS = {"A": [1, 6, 23, 70], "B": [2, 9, 41, 130], "C": [3, 64, 150, 333], "D": [1, 2, 17, 45]}


def _folder(tmp_path, name, dtype, std=0.08):
    cfg, seed, _ = CONFIGS[name]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    return H.make_folder(tmp_path / f"f{name}_{dtype}", cfg, seed, dtype=stored, std=std)


def _engine(folder, dtype, page_size, num_pages, max_requests=8):
    from batchspec_b200.engine import Engine
    eng = Engine(dtype=dtype, device=DEV)
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=max_requests, page_size=page_size, num_pages=num_pages)
    return eng


def _oracle(folder, tokens):
    cfg, w = P.read_model_folder(folder)
    return P.forward(cfg, w, tokens)[0].numpy()


def _compare(got, folder, reqs, dtype):
    """Every row against the oracle.  float32: no row beyond the tolerance.  bfloat16: one row in fifty, or one, may
    be (a router's choice between two experts whose logits differ by less than the rounding falls either way), none
    beyond three times the tolerance... unless the router chose differently, which the share bounds."""
    bf = dtype == "bfloat16"
    return H.compare_with_oracle(got, folder, reqs, dtype, oracle=_oracle, allow_over=0.03 if bf else 0.0,
                                 allow_rows=1 if bf else 0)


def _requests(name):
    cfg, seed, _ = CONFIGS[name]
    return {f"r{i}": H.random_tokens(n, cfg["vocab"], 100 * seed + i) for i, n in enumerate(LENGTHS[name])}


def _rows_agree(a, b, dtype, share=0.03):
    bad = [k for k in a if np.abs(a[k] - b[k]).max() > H.TOL[dtype] * np.abs(a[k]).max()]
    assert len(bad) <= (max(1, share * len(a)) if dtype == "bfloat16" else 0), bad[:5]


@pytest.fixture(scope="module")
def ops():
    from batchspec_b200.kernels import ops as o
    o.load_library()
    return o


# ---------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,S,d", [(3, 4, 96), (5, 1, 50), (2, 3, 4096), (1, 16, 30), (4, 2, 7)])
def test_streams_join_read_norm_and_sum(ops, dtype, n, S, d):
    """x_t <- sum_s mix[s, t] x_s + out[t] (vec * y); u = sum_s in[s] x_s normalised with 1 + w; the final sum."""
    g = torch.Generator(device=DEV).manual_seed(n * 100 + S)
    src = torch.randn(n, d, device=DEV, generator=g)
    x = ops.stream_expand(src, S)
    assert all(torch.equal(x[:, s], src) for s in range(S))
    x = x + 0.3 * torch.randn(n, S, d, device=DEV, generator=g)
    y = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    vec = 1 + 0.2 * torch.randn(d, device=DEV, generator=g)
    mix = torch.eye(S, device=DEV) + 0.3 * torch.randn(S, S, device=DEV, generator=g)
    out_c, in_c = torch.randn(S, device=DEV, generator=g), torch.randn(S, device=DEV, generator=g)
    w = 0.2 * torch.randn(d, device=DEV, generator=g)
    mixw = torch.cat([mix.reshape(-1), out_c]).contiguous()
    eps = 1e-5
    xs = [x[:, s].double() for s in range(S)]
    yy = vec.double() * y.double()
    new = [sum(mix[j, t].double() * xs[j] for j in range(S)) + out_c[t].double() * yy for t in range(S)]
    u = sum(in_c[t].double() * new[t] for t in range(S))
    want = P.one_plus_norm(u, w, eps)
    rows = torch.tensor(list(range(n - 1, -1, -1)), dtype=torch.int32, device=DEV)
    picked = torch.empty(n, d, device=DEV)
    ops.stream_gather(x, y, vec, mixw, rows, picked)            # leaves x as it is
    assert (picked.double() - sum(new)[rows.long()]).abs().max() <= 1e-5 * (1 + sum(new).abs().max())
    got = torch.empty(n, d, device=DEV, dtype=dtype)
    ops.stream_norm(x, y, vec, mixw, in_c, (1 + w).contiguous(), eps, got)
    for t in range(S):
        assert (x[:, t].double() - new[t]).abs().max() <= 1e-5 * (1 + new[t].abs().max())
    assert (got.double() - want).abs().max() <= (2e-5 if dtype == torch.float32 else 2e-2) * (1 + want.abs().max())
    before = x.clone()                                           # nothing pending: read and norm only
    ops.stream_norm(x, None, None, None, in_c, (1 + w).contiguous(), eps, got)
    assert torch.equal(x, before)
    want2 = P.one_plus_norm(sum(in_c[t].double() * before[:, t].double() for t in range(S)), w, eps)
    assert (got.double() - want2).abs().max() <= (2e-5 if dtype == torch.float32 else 2e-2) * (1 + want2.abs().max())
    ops.stream_gather(x, None, None, None, rows, picked)
    assert (picked.double() - before.double().sum(1)[rows.long()]).abs().max() <= 1e-5 * (1 + before.abs().max() * S)
    # a step's first norm fills the streams from the embedding rows itself: the same as expanding first
    filled = torch.full((n, S, d), float("nan"), device=DEV)
    got_fill = torch.empty(n, d, device=DEV, dtype=dtype)
    ops.stream_norm(filled, None, None, None, in_c, (1 + w).contiguous(), eps, got_fill, expand=src)
    expanded = ops.stream_expand(src, S)
    ops.stream_norm(expanded, None, None, None, in_c, (1 + w).contiguous(), eps, got)
    assert torch.equal(filled, expanded) and torch.equal(got_fill, got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_squared_relu_feed_forward(ops, dtype):
    from batchspec_b200.parts.base import FEED_FORWARDS, PartSpec, Runtime, build_part
    g = torch.Generator(device=DEV).manual_seed(3)
    # rows up to 8 with inner sizes that are multiples of 8 take the product with the activation in its epilogue
    for n, d, ff in ((5, 48, 40), (1, 100, 44), (70, 320, 192), (1, 512, 1024), (8, 320, 200), (3, 2048, 8448), (9, 512, 1024)):
        part = build_part(FEED_FORWARDS, PartSpec("mlp", dict(dim=d, intermediate=ff)), Runtime(dtype, torch.device(DEV)))
        w = {"up": (0.2 * torch.randn(ff, d, device=DEV, generator=g)).to(dtype),
             "down": (0.2 * torch.randn(d, ff, device=DEV, generator=g)).to(dtype)}
        part.bind(w)
        x = torch.randn(n, d, device=DEV, generator=g).to(dtype)
        want = P.squared_relu_mlp(x.double().cpu(), {k: v.cpu() for k, v in w.items()})
        got = part.forward(x, None).double().cpu()
        assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,d,ff,E,top", [(7, 48, 16, 5, 2), (1, 100, 20, 7, 7), (40, 64, 32, 1, 1), (300, 320, 96, 12, 3),
                                          (3, 320, 64, 8, 2), (70, 64, 128, 16, 3), (210, 320, 16, 4, 1), (600, 96, 40, 3, 2),
                                          (9, 256, 96, 2, 2), (2000, 128, 64, 8, 4)])
def test_routed_gated_experts_with_softmax_over_the_chosen(ops, dtype, n, d, ff, E, top):
    """The router's logits are spread so that no choice is close; the weights are the softmax over the chosen logits
    alone, which the bias (large for one expert) shows: that expert is always chosen."""
    from batchspec_b200.parts.base import FEED_FORWARDS, PartSpec, Runtime, build_part
    g = torch.Generator(device=DEV).manual_seed(n + E)
    part = build_part(FEED_FORWARDS, PartSpec("routed_glu", dict(dim=d, intermediate=ff, n_experts=E, top=top)),
                      Runtime(dtype, torch.device(DEV)))
    w = {"router": (torch.randn(E, d, device=DEV, generator=g) / math.sqrt(d)).to(dtype),
         "router_bias": (torch.randn(E, device=DEV, generator=g) + 6.0 * (torch.arange(E, device=DEV) == E - 1)).to(dtype)}
    for e in range(E):
        w[f"gate{e}"] = (0.3 * torch.randn(ff, d, device=DEV, generator=g)).to(dtype)
        w[f"up{e}"] = (0.3 * torch.randn(ff, d, device=DEV, generator=g)).to(dtype)
        w[f"down{e}"] = (0.3 * torch.randn(d, ff, device=DEV, generator=g)).to(dtype)
    part.bind(w)
    x = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    ids, wts = ops.moe_route(x, part.w_router, part.b_router, 1, 1, top, 1.0, softmax_top=True)
    idx, wt = P.route(x.double().cpu(), w["router"].cpu(), w["router_bias"].cpu(), top)
    z = x.double().cpu() @ w["router"].double().cpu().T + w["router_bias"].double().cpu()
    srt = torch.sort(z, dim=-1, descending=True).values
    clear = torch.ones(n, dtype=torch.bool) if top == E else (srt[:, top - 1] - srt[:, top]) > 0.05
    assert clear.float().mean() > 0.7
    assert torch.equal(torch.sort(ids.cpu().long()[clear], dim=-1).values, torch.sort(idx[clear], dim=-1).values)
    assert (ids.cpu() == E - 1).any(dim=-1)[clear].all() or E == 1
    assert (wts.sum(-1) - 1).abs().max() <= 1e-5
    named = {"router": w["router"].cpu(), "router.b": w["router_bias"].cpu()}
    for e in range(E):
        named.update({f"e{e}.gate": w[f"gate{e}"].cpu(), f"e{e}.up": w[f"up{e}"].cpu(), f"e{e}.down": w[f"down{e}"].cpu()})
    want = P.routed_experts(x.double().cpu(), named, E, top)
    got = part.forward(x, None).double().cpu()
    err = (got - want).abs().amax(dim=-1) / want.abs().max()
    assert err[clear].max() <= (2e-5 if dtype == torch.float32 else 3e-2)


def _latent_case(ops, dtype, H_, R, Pd, ps, q_lens, kv_lens, window, sink, spike=None, seed=0, generic=False,
                 drop_passed_pages=True, with_entries=False):
    """Random queries and entries, pages in scrambled order, a window and a sink logit per head; the table entries of
    pages that the window has passed for every query are -1, as after the cache gave them back.  (got, want) [n, H, R]."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    n = sum(q_lens)
    ql = torch.randn(H_, n, R, device=DEV, generator=g)
    qr = torch.randn(n, H_, Pd, device=DEV, generator=g)
    ents = [torch.randn(L, R + Pd, device=DEV, generator=g) for L in kv_lens]
    sinks = (2.0 * torch.randn(H_, device=DEV, generator=g)) if sink else None
    if spike is not None:                      # one key whose score would take all of one query's softmax if seen
        e, key, head = spike
        t = sum(q_lens[:e]) + q_lens[e] - 1
        ql[head, t] = 0
        qr[t, head] = 0
        qr[t, head, Pd - 1] = 40.0
        ents[e][:, R + Pd - 1].clamp_(-1, 1)
        ents[e][key, R + Pd - 1] = 30.0
    ql, qr, ents = ql.to(dtype), qr.to(dtype), [x.to(dtype) for x in ents]
    pages_per = [-(-L // ps) for L in kv_lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(seed + 1))[:sum(pages_per)]
    cache = torch.randn(n_pages, 1, ps * (R + Pd), device=DEV, generator=g).to(dtype)
    indptr = [0] + list(np.cumsum(pages_per))
    table = perm.clone()
    for e, L in enumerate(kv_lens):
        for p in range(L):
            cache[int(perm[indptr[e] + p // ps]), 0].view(ps, R + Pd)[p % ps] = ents[e][p]
        if window and drop_passed_pages:
            first_needed = max(0, (L - q_lens[e]) - window + 1)       # what the first query of the portion still sees
            table[indptr[e]:indptr[e] + first_needed // ps] = -1
    qo = [0] + list(np.cumsum(q_lens))
    pos = torch.cat([torch.arange(L - q, L) for q, L in zip(q_lens, kv_lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(DEV, torch.int32)
    ctx = SimpleNamespace(qo_indptr=torch.tensor(qo, dtype=torch.int32, device=DEV), positions=pos, tok_entry=ent,
                          n_entries=len(q_lens), n_tokens=n, max_q_len=max(q_lens), max_kv_len=max(kv_lens),
                          kv_len=torch.tensor(kv_lens, dtype=torch.int32, device=DEV),
                          extras={"min_q_len": min(q_lens)})
    tables = SimpleNamespace(kv_indptr=torch.tensor(indptr, dtype=torch.int32, device=DEV),
                             kv_indices=table.to(DEV, torch.int32), page_size=ps)
    out = torch.full((H_, n, R), float("nan"), device=DEV, dtype=dtype)
    scale = 0.5 / math.sqrt(R + Pd)
    ops.FORCE_GENERIC_LATENT = generic
    try:
        ops.latent_attention(ql, qr, out, cache, ctx, tables, H_, R, Pd, scale, window=window or 0, sink=sinks)
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        ops.FORCE_GENERIC_LATENT = False
    want = torch.empty(n, H_, R, device=DEV, dtype=F64)
    for e, (q, L) in enumerate(zip(q_lens, kv_lens)):
        x = ents[e].double()
        for i in range(q):
            p, t = L - q + i, qo[e] + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(H_):
                s = (x[lo:p + 1] @ torch.cat([ql[h, t].double(), qr[t, h].double()])) * scale
                if sink:
                    s = torch.cat([s, sinks[h].double().reshape(1)])
                w = torch.softmax(s, 0)
                want[t, h] = w[:p + 1 - lo] @ x[lo:p + 1, :R]
    if with_entries:
        return out.double().transpose(0, 1), want, ents
    return out.double().transpose(0, 1), want


LATENT_WINDOW_SHAPES = [
    # heads, latent, rotated, page, q_lens, kv_lens, window
    (3, 48, 8, 4, [5, 1, 2], [5, 9, 30], 7),
    (1, 20, 4, 1, [1, 1, 7], [40, 1, 7], 1),
    (5, 72, 16, 5, [3, 11], [17, 11], 100),
    (16, 128, 32, 16, [1, 1, 1, 1], [300, 17, 64, 129], 64),
    (16, 128, 32, 16, [70, 2, 1], [200, 5, 333], 33),
    (6, 112, 16, 16, [130, 1, 3, 64], [130, 555, 40, 600], 96),
    (8, 96, 16, 16, [1, 1, 1], [5, 130, 64], 96),
    (8, 96, 16, 16, [97, 40], [97, 300], 96),
    (32, 160, 32, 16, [1, 1], [1300, 31], 1000),
    (4, 64, 16, 8, [33, 1], [33, 2049], None),           # a sink without a window
    (16, 512, 64, 16, [1, 1, 40], [700, 65, 300], 128),  # the widest latent the tensor-core kernel takes
    (128, 256, 64, 64, [1, 2], [700, 65], 500),
]


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", LATENT_WINDOW_SHAPES, ids=lambda s: f"H{s[0]}r{s[1]}p{s[2]}ps{s[3]}w{s[6]}")
def test_latent_attention_with_window_and_sink(ops, dtype, shape, generic):
    if generic and dtype == torch.float32:
        pytest.skip("float32 always runs the generic kernel")
    Hh, R, Pd, ps, q_lens, kv_lens, window = shape
    got, want = _latent_case(ops, dtype, Hh, R, Pd, ps, q_lens, kv_lens, window, True, generic=generic)
    assert not torch.isnan(got).any()
    assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else 2.5e-2)


def test_the_sink_takes_its_share_of_the_weight(ops):
    """With scores near zero over 3 keys and a sink logit of ln 5, the output is 3/8 of the keys' mean."""
    Hh, R, Pd, ps = 2, 32, 16, 4
    for dtype, generic in ((torch.float32, True), (torch.bfloat16, False), (torch.bfloat16, True)):
        ents = torch.randn(3, R + Pd, device=DEV).to(dtype)
        cache = torch.zeros(2, 1, ps * (R + Pd), device=DEV, dtype=dtype)
        cache[1, 0].view(ps, R + Pd)[:3] = ents
        ctx = SimpleNamespace(qo_indptr=torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                              positions=torch.tensor([2], dtype=torch.int32, device=DEV), n_entries=1, n_tokens=1,
                              max_q_len=1, max_kv_len=3, extras={})
        tables = SimpleNamespace(kv_indptr=torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                 kv_indices=torch.tensor([1], dtype=torch.int32, device=DEV), page_size=ps)
        out = torch.empty(Hh, 1, R, device=DEV, dtype=dtype)
        sinks = torch.tensor([math.log(5.0), -1e4], device=DEV)
        ops.FORCE_GENERIC_LATENT = generic
        try:
            ops.latent_attention(torch.zeros(Hh, 1, R, device=DEV, dtype=dtype), torch.zeros(1, Hh, Pd, device=DEV, dtype=dtype),
                                 out, cache, ctx, tables, Hh, R, Pd, 1.0, window=0, sink=sinks)
        finally:
            ops.FORCE_GENERIC_LATENT = False
        mean = ents[:, :R].float().mean(0)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert (out[0, 0].float() - 3.0 / 8.0 * mean).abs().max() <= tol
        assert (out[1, 0].float() - mean).abs().max() <= tol      # a sink far below every score counts for nothing


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("back", [0, 1, 15, 16, 94, 95, 96, 97, 111, 112, 200, 500])
def test_one_latent_key_decides_inside_the_window_and_is_unseen_outside(ops, dtype, back, generic):
    """A key ``back`` positions before the query whose score would take the whole softmax: with a window of 96 it
    does for back <= 95 (the window's last key, page borders, the query's own) and leaves no trace from 96 on; from a
    decoded token and from the last token of a portion."""
    if generic and dtype == torch.float32:
        pytest.skip("float32 always runs the generic kernel")
    L = 640
    for q_lens in ([1, 1], [3, 70]):
        got, want, ents = _latent_case(ops, dtype, 8, 96, 16, 16, q_lens, [90, L], 96, True, spike=(1, L - 1 - back, 5),
                                       seed=back, generic=generic, with_entries=True)
        t = sum(q_lens) - 1
        tol = 2e-5 if dtype == torch.float32 else 2.5e-2
        assert (got[t, 5] - want[t, 5]).abs().max() <= 5 * tol
        assert (got - want).abs().max() <= 5 * tol
        # the edge shows in the result: the spiked key's latent is the output inside the window only
        spiked = ents[1][L - 1 - back, :96].double()
        assert ((got[t, 5] - spiked).abs().max() <= 5 * tol) == (back <= 95)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,G,hd,vd,rot,ps", [(4, 2, 12, 20, 8, 4), (8, 1, 64, 64, 16, 16), (3, 3, 16, 5, 0, 8),
                                               (6, 3, 8, 12, 8, 4), (2, 1, 128, 128, 128, 16)])
def test_weighted_head_norm_before_the_rotation_by_halves(ops, dtype, Hq, G, hd, vd, rot, ps):
    """q and k heads: RMS norm with a weight shared by the heads, then the rotation of the first ``rot`` numbers in
    the (i, i + rot/2) pairing; v untouched; k and v land in the pages of their positions."""
    g = torch.Generator(device=DEV).manual_seed(Hq * 10 + hd)
    lens, starts = [3, 1, 9], [0, 6, 2]
    n = sum(lens)
    eps, base = 1e-5, 500.0
    width = (Hq + G) * hd + G * vd
    qkv = torch.randn(n, width + 3, device=DEV, generator=g) * 2
    wq = (1 + 0.3 * torch.randn(hd, device=DEV, generator=g)).to(dtype)
    wk = (1 + 0.3 * torch.randn(hd, device=DEV, generator=g)).to(dtype)
    pos = torch.cat([torch.arange(s, s + k) for s, k in zip(starts, lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((k,), i) for i, k in enumerate(lens)]).to(DEV, torch.int32)
    pages_per = [-(-(s + k) // ps) for s, k in zip(starts, lens)]
    indptr = torch.tensor([0] + list(np.cumsum(pages_per)), dtype=torch.int32, device=DEV)
    idx = torch.randperm(sum(pages_per), generator=torch.Generator().manual_seed(1)).to(DEV, torch.int32)
    cache = torch.zeros(sum(pages_per), 1, ps * G * (hd + vd), device=DEV, dtype=dtype)
    freqs, mag = P.yarn_frequencies(base, rot, None) if rot else ([], 1.0)
    table = ops.rope_frequency_table(torch.tensor(freqs, dtype=F64), DEV) if rot else None
    q = ops.qkv_prepare(qkv[:, :width], Hq, G, hd, vd, None, table, rot, False, mag, eps, pos, ent, indptr, idx, cache, ps,
                        q_norm=wq, k_norm=wk, norm_first=True)
    x = qkv.double().cpu()
    qq = P.weighted_norm(x[:, :Hq * hd].view(n, Hq, hd), wq.cpu(), eps)
    kk = P.weighted_norm(x[:, Hq * hd:(Hq + G) * hd].view(n, G, hd), wk.cpu(), eps)
    if rot:
        qq, kk = P.rotate(qq, pos.tolist(), freqs, mag, False), P.rotate(kk, pos.tolist(), freqs, mag, False)
    vv = x[:, (Hq + G) * hd:width].view(n, G, vd)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (q.double().cpu().view(n, Hq, hd) - qq).abs().max() <= tol * qq.abs().max()
    for t in range(n):
        e, p = int(ent[t]), int(pos[t])
        page = cache[int(idx[int(indptr[e]) + p // ps]), 0].double().cpu()
        k_rows = page[:G * ps * hd].view(G, ps, hd)[:, p % ps]
        v_rows = page[G * ps * hd:].view(G, ps, vd)[:, p % ps]
        assert (k_rows - kk[t]).abs().max() <= tol * kk.abs().max()
        assert (v_rows - vv[t]).abs().max() <= tol * vv.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(4, 2, 12, 20, 8), (8, 1, 64, 64, 16), (3, 3, 10, 4, 10), (8, 2, 128, 128, 64)],
                         ids=lambda s: f"H{s[0]}G{s[1]}d{s[2]}v{s[3]}")
def test_attention_mixer_with_head_norms_and_a_gate_per_head(ops, dtype, sizes):
    """The whole mixer (projections, weighted head norms, rotation, causal softmax over grouped heads, one gate per
    head, output projection) on a prompt and then token by token, against the plain function; heads of 64 and 128
    with values as wide run the tensor-core kernels in bfloat16."""
    Hq, G, hd, vd, rot = sizes
    d, page = 96, 8
    layer = _attn(Hq, G, hd, vd, 1.0 / math.sqrt(hd), rot_dims=rot, base=777.0)
    cfg = _config(50, d, 1e-5, [layer])
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    _one_mixer_against_plain(cfg, dtype, stored, page, P.gated_attention, lens=(37, 90))


@pytest.mark.parametrize("kind", ["attention", "latent", "latent_window"])
def test_one_key_among_hundreds_takes_the_softmax(ops, kind):
    """With a scale far above 1 / sqrt(size) the scores spread over tens of units and one key, wherever it lies among
    the hundreds before a query (the first token, page borders, far back, the query's own), takes nearly all of the
    softmax: a key that a kernel skipped or misplaced would change the whole output.  float32, prompt and decoding."""
    if kind == "attention":
        layer, plain = _attn(4, 2, 32, 24, 4.0, rot_dims=16, base=777.0), P.gated_attention
    else:
        layer = _latent(4, 16, 8, 24, 32, 48, 3.0, 3000.0, window=70 if kind == "latent_window" else None)
        plain = P.latent_attention
    _one_mixer_against_plain(_config(50, 96, 1e-5, [layer]), "float32", torch.float32, 8, plain, lens=(9, 300),
                             peaky=True)


def _one_mixer_against_plain(cfg, dtype, stored, page, plain, lens, peaky=False):
    """Build the model's only mixer with random tensors and run it through the step context of a real engine."""
    import tempfile
    from batchspec_b200.engine import StepEntry
    with tempfile.TemporaryDirectory() as tmp:
        folder = H.make_folder(tmp, cfg, 5, dtype=stored, std=0.25)
        _, w = P.read_model_folder(folder)
        eng = _engine(folder, dtype, page, 64, max_requests=2)
        block = eng.model.blocks[0]
        seen = {}
        real = block.mixer.forward

        def spy(x, ctx, cache):
            out = real(x, ctx, cache)
            seen.setdefault("x", []).append(x.detach().double().cpu())
            seen.setdefault("y", []).append(out.detach().double().cpu())
            return out
        block.mixer.forward = spy
        for rid, n in zip("ab", lens):
            toks = H.random_tokens(n, cfg["vocab"], n)
            eng.admit(rid)
            head = n - 5
            eng.step([StepEntry(rid, toks[:head], [])])
            for t in toks[head:]:
                eng.step([StepEntry(rid, [t], [])])
            xs, ys = torch.cat(seen.pop("x")), torch.cat(seen.pop("y"))
            sub = {k[len("l0.mix."):]: v for k, v in w.items() if k.startswith("l0.mix.")}
            want = plain(xs, sub, cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
            err = (ys - want).abs().max() / want.abs().max()
            assert err <= ((1e-4 if peaky else 2e-5) if dtype == "float32" else 3e-2), (rid, float(err))
            if peaky and n > 100:         # the softmax is as sharp as the test wants: most queries have one key
                m = cfg["layers"][0]["mixer"]
                assert _largest_weights(xs, sub, m, cfg["norm"]["eps"]).median() > 0.9
            eng.release(rid)


def _largest_weights(h, w, m, eps):
    """The largest softmax weight of every (token, head) of a mixer, from the plain functions' own pieces."""
    T = h.shape[0]
    pos = list(range(T))
    if "kv_rank" in m:
        Hh, D, Pd, R = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
        q = (P.weighted_norm(h @ P.f64(w["dq"]).T, w["dq.norm"], eps) @ P.f64(w["uq"]).T).view(T, Hh, D + Pd)
        down = h @ P.f64(w["dkv"]).T
        c = P.weighted_norm(down[:, :R], w["dkv.norm"], eps)
        f, mag = P.yarn_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
        k = torch.cat([(c @ P.f64(w["uk"]).T).view(T, Hh, D),
                       P.rotate(down[:, R:].view(T, 1, Pd), pos, f, mag, True).expand(T, Hh, Pd)], dim=2)
        q = torch.cat([q[:, :, :D], P.rotate(q[:, :, D:], pos, f, mag, True)], dim=2)
        window = (m.get("mask") or {}).get("size")
    else:
        Hh, G, D = m["heads"], m["kv_heads"], m["dim"]
        q = P.weighted_norm((h @ P.f64(w["q"]).T).view(T, Hh, D), w["q.norm"], eps)
        k = P.weighted_norm((h @ P.f64(w["k"]).T).view(T, G, D), w["k.norm"], eps)
        f, mag = P.yarn_frequencies(m["rot"]["base"], m["rot"]["dims"], None)
        q, k = P.rotate(q, pos, f, mag, False), P.rotate(k, pos, f, mag, False).repeat_interleave(Hh // G, dim=1)
        window = None
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window else True)
    return torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1).amax(dim=-1)[:, 20:].flatten()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(3, 8, 4, 12, 20, 24, 10), (8, 32, 16, 48, 64, 96, 30), (1, 16, 8, 24, 8, 8, 1),
                                   (4, 64, 32, 64, 64, 128, None)], ids=lambda s: f"H{s[0]}r{s[5]}w{s[6]}")
def test_latent_mixer_with_window_and_sink(ops, dtype, sizes):
    Hh, dim, rot_dim, vdim, q_rank, kv_rank, window = sizes
    layer = _latent(Hh, dim, rot_dim, vdim, q_rank, kv_rank, 1.0 / math.sqrt(dim + rot_dim), 3000.0, window=window,
                    scaling=(3.0, 16, 8.0, 1.0))
    cfg = _config(50, 96, 1e-5, [layer])
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    _one_mixer_against_plain(cfg, dtype, stored, 8, P.latent_attention, lens=(37, 90))


# ---------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_tail_portions(tmp_path, name, dtype):
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    reqs = _requests(name)
    longest = max(len(t) for t in reqs.values())
    eng = _engine(folder, dtype, page, -(-longest // page) + 1)
    for rid, toks in reqs.items():
        one = {rid: toks}
        got = H.run_steps_in_process(eng, H.whole(rid, toks))
        _compare(got, folder, one, dtype)
        got_tail = H.run_steps_in_process(eng, H.tail_decoded(rid, toks, tail=40))
        _compare(got_tail, folder, one, dtype)
        got_port = H.run_steps_in_process(eng, H.portions(rid, toks, [7, 2, 16, 3, 2, 5, 2, 31]))
        _compare(got_port, folder, one, dtype)
        _rows_agree(got, got_tail, dtype)
        _rows_agree(got, got_port, dtype)
    assert all(g.pool.num_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_token_by_token_from_the_first_token(tmp_path, name, dtype):
    """A whole request decoded one token at a time (the first tokens of a sequence, every page border and window
    edge, long decoding) against the oracle."""
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    toks = H.random_tokens(150, cfg["vocab"], 4)
    eng = _engine(folder, dtype, page, 40)
    got = H.run_steps_in_process(eng, H.portions("t", toks, [1]))
    _compare(got, folder, {"t": toks}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_requests_reuse_pages(tmp_path, name, dtype):
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    base = _requests(name)
    reqs = dict(base)
    for i, (rid, toks) in enumerate(base.items()):          # twice as many requests as may be live
        reqs[f"s{i}"] = H.random_tokens(max(2, len(toks) // 2 + 3), cfg["vocab"], 999 + i)
    steps = H.mixed(reqs, seed=seed + 7, max_live=4)
    max_tokens = H.max_live_tokens(steps, round_to=page)
    eng = _engine(folder, dtype, page, max_tokens // page, max_requests=4)
    got = H.run_steps_in_process(eng, steps)
    _compare(got, folder, reqs, dtype)
    alone = _engine(folder, dtype, page, -(-max(len(t) for t in reqs.values()) // page) + 1)
    for rid in ("r2", "r3"):                                # every request alone gives the same rows as in the batch
        one = H.run_steps_in_process(alone, H.whole(rid, reqs[rid]))
        _rows_agree(one, {k: got[k] for k in one}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tmp_path, dtype):
    cfg, seed, page = CONFIGS["A"]
    folder = _folder(tmp_path, "A", dtype)
    reqs = _requests("A")
    steps = H.mixed(reqs, seed=3, max_live=4)
    got = H.run_trace_subprocess(folder, dtype, steps, tmp_path / "out", H.max_live_tokens(steps, round_to=64))
    _compare(got, folder, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_token_outside_the_window_is_unseen_and_the_first_inside_is_seen(tmp_path, dtype):
    """One latent layer, a window of 12 positions, four streams: changing a token that the window hides from the
    positions 36..47 changes none of their logits, bit for bit; changing the first token they see changes them.  As
    one prompt, token by token, and in portions that cross the edge inside a page."""
    cfg, seed, page = CONFIGS["WINDOW"]
    folder = _folder(tmp_path, "WINDOW", dtype, std=0.3)
    base = H.random_tokens(48, cfg["vocab"], 2)
    eng = _engine(folder, dtype, page, 12)
    # position 47 sees 36..47, position 36 sees 25..36
    cases = ((24, [], range(36, 48)), (25, [36], range(37, 48)), (35, range(36, 47), [47]), (0, [], range(36, 48)))
    for make in (lambda t: H.whole("e", t), lambda t: H.portions("e", t, [1]), lambda t: H.portions("e", t, [10, 3, 2, 9])):
        ref = H.run_steps_in_process(eng, make(base))
        _compare(ref, folder, {"e": base}, dtype)
        for where, moved, same in cases:
            toks = list(base)
            toks[where] = (toks[where] + 1) % cfg["vocab"]
            got = H.run_steps_in_process(eng, make(toks))
            for p in same:
                assert np.array_equal(got[("e", p)], ref[("e", p)]), (where, p)
            for p in moved:
                assert not np.array_equal(got[("e", p)], ref[("e", p)]), (where, p)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_decides_the_logits_through_full_attention(tmp_path, dtype):
    """Changing ONE token far back changes the last position's logits in the oracle although every window has passed
    it: the causal attention layers see it.  The engine follows, decoded alone and as the end of a portion."""
    cfg, seed, page = CONFIGS["A"]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = H.make_folder(tmp_path / "far", cfg, 21, dtype=stored, std=0.15)
    base = H.random_tokens(260, cfg["vocab"], 8)
    eng = _engine(folder, dtype, page, 70)
    ref0 = _oracle(folder, base)[-1]
    moved = []
    for where in (0, 3, 4, 127, 128, 200):
        toks = list(base)
        toks[where] = (toks[where] + 17) % cfg["vocab"]
        ref = _oracle(folder, toks)
        moved.append(np.abs(ref[-1] - ref0).max() / np.abs(ref0).max())
        for steps in (H.tail_decoded("f", toks, tail=3), H.portions("f", toks, [250, 10])):
            got = H.run_steps_in_process(eng, steps)
            err = np.abs(got[("f", len(toks) - 1)] - ref[-1]).max() / np.abs(ref).max()
            assert err <= H.TOL[dtype] * (1 if dtype == "float32" else 2), (where, err)
    assert max(moved) > 1e-3, "no far token moved the last logits: the weights hide what this test is for"


def test_generation_through_the_scheduler(tmp_path):
    """Greedy generation through Engine.generate (scheduler, portions, captured decode steps) gives the tokens that
    the oracle's argmax gives, token by token, for requests of unequal length under page pressure."""
    from batchspec_b200.engine import Engine
    from batchspec_b200.engine.sequence import Sequence
    cfg, seed, page = CONFIGS["A"]
    folder = H.make_folder(tmp_path / "gen", cfg, 31, dtype=torch.float32, std=0.2)
    prompts = [H.random_tokens(n, cfg["vocab"], 50 + n) for n in (3, 19, 42, 7, 64)]
    for graphs in (True, False):
        eng = Engine(dtype="float32", device=DEV)
        eng.load_model(model_dir=folder)
        eng.use_cuda_graphs = graphs
        eng.setup_caches(max_batch_size=3, max_seq_length=96, page_size=page, prefill_chunk_size=16, num_pages=70)
        eng.setup_sampling_params(temperature=0.0)
        seqs = [Sequence(i, list(p), max_new_tokens=12) for i, p in enumerate(prompts)]
        done = {s.seq_id: s for s in eng.generate(seqs)}
        for i, p in enumerate(prompts):
            toks = list(p)
            for k in range(12):
                ref = _oracle(folder, toks)[-1]
                top2 = np.sort(ref)[-2:]
                nxt = done[i].output_ids[k]
                if top2[1] - top2[0] > 1e-3 * np.abs(ref).max():
                    assert nxt == int(ref.argmax()), (graphs, i, k)
                toks.append(nxt)
