"""The Tokolorn design on the engine against the plain implementation in ``plain_tokolorn.py``: every mechanism alone
(kernels against one plain function each), then whole models of three configurations that share no size, fed whole,
with a decoded tail, in portions down to two tokens, token by token, in mixed batches over pools that force pages and
slots to be used again, through ``bin/trace_run`` and through the scheduler."""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers as H
import plain_tokolorn as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
F64 = torch.float64


def _lightning(heads, dim, vdim, decay, ff=None):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def _parallel(heads, kv_heads, dim, vdim, scale, window, rot_dims, base, softcap, inner, state, dt_rank, conv,
              left_scale, right_scale, ff=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap)
    if window:
        left["mask"] = dict(size=window)
    if rot_dims:
        left["rot"] = dict(base=base, dims=rot_dims)
    return dict(type="parallel", mixer=dict(left=left, right=dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv),
                                            left_scale=left_scale, right_scale=right_scale),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def _attention(heads, kv_heads, dim, scale, chunk, ff=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if chunk:
        m["mask"] = dict(size=chunk)
    return dict(type="attention", mixer=m, mlp=dict(kind="dense", ff=ff) if ff else None)


def _config(vocab, width, eps, layers, loop=None, bigram=(61, 5, 3), embed_scale=3.0, logit_scale=0.7):
    emb = dict(scale=embed_scale)
    if bigram:
        emb["bigram"] = dict(buckets=bigram[0], mul_prev=bigram[1], mul_cur=bigram[2])
    cfg = dict(architecture="Tokolorn", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale,
               embedding=emb, layers=layers)
    if loop:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


# Three configurations that share no size.  A: a loop from layer 0, a layer without a feed-forward, a window that is
# no multiple of the page, rotation of a part of the head.  B: a loop in the middle, odd sizes (width 100, key size 6,
# one tap, 40 states), no window, no chunk.  C: sizes at which the products' fused epilogues, 8-wide loads and, in
# bfloat16, the tensor-core attention kernels run (heads of 64 for keys and values).
CFG_A = _config(200, 48, 1e-5, [_lightning(3, 8, 12, (0.5, 0.9, 0.99), ff=40),
                                _parallel(4, 2, 12, 20, 0.3, 10, 8, 5000.0, 5.0, 24, 5, 3, 3, 0.6, 0.5),
                                _attention(3, 3, 16, 0.25, 12, ff=56)], loop=(0, 2, 2))
CFG_B = _config(513, 100, 1e-6, [_attention(2, 1, 6, 0.4, None, ff=36),
                                 _lightning(2, 20, 7, (0.8, 0.999), ff=36),
                                 _parallel(3, 3, 10, 10, 0.3, None, None, None, None, 36, 40, 7, 1, 1.0, 1.5, ff=44),
                                 _lightning(1, 6, 40, (0.95,))], loop=(1, 3, 2), bigram=(17, 1000003, 1), embed_scale=1.0,
                logit_scale=1.0)
CFG_C = _config(640, 320, 1e-5, [_parallel(8, 2, 64, 64, 0.125, 128, 64, 100000.0, 25.0, 128, 16, 8, 4, 0.7, 0.4, ff=192),
                                 _lightning(5, 64, 64, (0.7, 0.9, 0.97, 0.999, 0.8), ff=192),
                                 _attention(8, 4, 64, 0.125, 64, ff=192)])
# one layer each, no bigram rows: a changed token reaches other positions through the mixer alone
CFG_WINDOW = _config(150, 32, 1e-5, [_parallel(2, 1, 16, 8, 0.5, 12, 16, 1000.0, 8.0, 8, 4, 2, 2, 1.0, 0.0, ff=24)],
                     bigram=None)
CFG_CHUNK = _config(150, 32, 1e-5, [_attention(2, 1, 16, 0.5, 12, ff=24)], bigram=None)
CFG_STATE = _config(90, 40, 1e-5, [_lightning(2, 16, 16, (0.9, 0.999), ff=24), _lightning(4, 8, 24, (0.5, 0.6, 0.7, 1.0))],
                    loop=(0, 1, 2))
CONFIGS = {"A": (CFG_A, 11, 4), "B": (CFG_B, 12, 8), "C": (CFG_C, 13, 16), "WINDOW": (CFG_WINDOW, 14, 8),
           "CHUNK": (CFG_CHUNK, 15, 8), "STATE": (CFG_STATE, 16, 4)}
LENGTHS = {"A": [1, 6, 23, 70], "B": [2, 9, 41, 130], "C": [3, 64, 150, 333]}


def _folder(tmp_path, name, dtype, std=0.08):
    cfg, seed, _ = CONFIGS[name]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    return H.make_folder(tmp_path / f"t{name}_{dtype}", cfg, seed, dtype=stored, std=std)


def _engine(folder, dtype, page_size, num_pages, max_requests=8):
    from batchspec_b200.engine import Engine
    eng = Engine(dtype=dtype, device=DEV)
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=max_requests, page_size=page_size, num_pages=num_pages)
    return eng


def _oracle(folder, tokens):
    cfg, w = P.read_model_folder(folder)
    return P.forward(cfg, w, tokens).numpy()


def _compare(got, folder, reqs, dtype):
    """Every row against the oracle.  float32: no row beyond the tolerance.  bfloat16: one row in fifty, or one, may
    be (the error is taken against the largest logit; a few dozen roundings of 2^-9 per row, through dot products of
    six terms that cancel, leave single rows at two or three times the typical error), none beyond three times the
    tolerance."""
    bf = dtype == "bfloat16"
    worst = H.compare_with_oracle(got, folder, reqs, dtype, oracle=_oracle, allow_over=0.02 if bf else 0.0,
                                  allow_rows=1 if bf else 0)
    assert worst[0] <= 3 * H.TOL[dtype], worst
    return worst


def _requests(name):
    cfg, seed, _ = CONFIGS[name]
    return {f"r{i}": H.random_tokens(n, cfg["vocab"], 100 * seed + i) for i, n in enumerate(LENGTHS[name])}


def _rows_agree(a, b, dtype):
    for k in a:
        assert np.abs(a[k] - b[k]).max() <= H.TOL[dtype] * np.abs(a[k]).max(), k


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


@pytest.fixture(scope="module")
def ops():
    from batchspec_b200.kernels import ops as o
    o.load_library()
    return o


def _i32(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def _step_ctx(lens, slots, positions=None, token_ids=None):
    ent = torch.cat([torch.full((k,), i) for i, k in enumerate(lens)]).to(DEV, torch.int32)
    return SimpleNamespace(qo_indptr=_i32([0] + list(np.cumsum(lens))), n_entries=len(lens), tok_entry=ent,
                           state_slots=_i32(slots), positions=positions, token_ids=token_ids, n_tokens=sum(lens))


# ------------------------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,d", [(3, 96), (5, 50), (2, 4096), (1, 18000)])
def test_norm_with_one_number_and_branches_scaled_by_column(ops, dtype, n, d):
    g = torch.Generator(device=DEV).manual_seed(d)
    resid = torch.randn(n, d, device=DEV, generator=g) * 3
    delta = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    vec = 1 + 0.5 * torch.randn(d, device=DEV, generator=g)
    w = torch.tensor([1.37], device=DEV).to(dtype)
    x = resid.double().cpu() + vec.double().cpu() * delta.double().cpu()
    want = P.scalar_norm(x, w.cpu(), 1e-5)
    r = resid.clone()
    out = torch.empty(n, d, device=DEV, dtype=dtype)
    ops.add_rmsnorm(r, delta, w, 1e-5, out, 1.0, True, vec)
    assert (r.double().cpu() - x).abs().max() <= 1e-6 * x.abs().max()
    assert (out.double().cpu() - want).abs().max() <= _tol(dtype) * want.abs().max()
    rows = _i32([n - 1, 0])
    picked = torch.empty(2, d, device=DEV)
    ops.gather_rows_add(resid, delta, rows, picked, 1.0, vec)
    assert (picked.double().cpu() - x[[n - 1, 0]]).abs().max() <= 1e-6 * x.abs().max()
    r2 = resid.clone()
    ops.residual_update(r2, delta, 1.0, vec=vec)
    assert (r2.double().cpu() - x).abs().max() <= 1e-6 * x.abs().max()


@pytest.mark.parametrize("M,I,K", [(1, 80, 64), (8, 448, 256), (5, 176, 72), (40, 256, 96), (3, 52, 64)])
def test_gelu_gate_in_the_product_and_alone(ops, M, I, K):
    g = torch.Generator(device=DEV).manual_seed(M * I)
    x = torch.randn(M, K, device=DEV, generator=g)
    wg, wu = torch.randn(I, K, device=DEV, generator=g) * 0.3, torch.randn(I, K, device=DEV, generator=g) * 0.3
    for dtype in (torch.float32, torch.bfloat16):
        xd, wgd, wud = x.to(dtype), wg.to(dtype), wu.to(dtype)
        want = P.gelu_tanh(xd.double().cpu() @ wgd.double().cpu().T) * (xd.double().cpu() @ wud.double().cpu().T)
        u = ops.linear(xd, torch.cat([wgd, wud]).contiguous())
        out = torch.empty(M, I, device=DEV, dtype=dtype)
        ops.gelu_tanh_mul(u, out)
        assert (out.double().cpu() - want).abs().max() <= _tol(dtype) * want.abs().max()
        if dtype == torch.bfloat16 and I % ops.GLU_GROUP == 0:
            got = ops.linear_glu(xd, ops.interleave_gate_up(wgd, wud), ops.GLU_GROUP, "gelu_tanh")
            assert (got.double().cpu() - want).abs().max() <= _tol(dtype) * want.abs().max()
    ops.check_status()


@pytest.mark.parametrize("buckets,mul_prev,mul_cur,vocab", [(61, 5, 3, 200), (1, 7, 7, 50), (499, 2000000011, 1999999973, 70000)])
def test_bigram_rows_over_portions_and_a_slot_used_again(ops, buckets, mul_prev, mul_cur, vocab):
    d = 24
    g = torch.Generator(device=DEV).manual_seed(buckets)
    table = torch.randn(buckets + 1, d, device=DEV, generator=g)
    emb = torch.zeros(vocab, d, dtype=F64)
    prev = torch.zeros(4, 1, dtype=torch.int32, device=DEV)
    toks = {"a": H.random_tokens(9, vocab, 1), "b": H.random_tokens(5, vocab, 2)}
    toks["a"][0] = toks["b"][1] = vocab - 1
    slots, at, got = {"a": 3, "b": 1}, {"a": 0, "b": 0}, {"a": [], "b": []}
    for step in (dict(a=1, b=2), dict(a=4), dict(b=1, a=1), dict(a=3, b=2)):
        lens = list(step.values())
        ids = [t for r, k in step.items() for t in toks[r][at[r]:at[r] + k]]
        pos = [p for r, k in step.items() for p in range(at[r], at[r] + k)]
        ctx = _step_ctx(lens, [slots[r] for r in step], _i32(pos), _i32(ids))
        resid = torch.zeros(len(ids), d, device=DEV)
        ops.bigram_add(resid, table, prev, ctx, buckets, mul_prev, mul_cur, vocab)
        o = 0
        for r, k in step.items():
            got[r].append(resid[o:o + k])
            at[r] += k
            o += k
    for r in toks:
        want = P.embed_rows(toks[r], emb, table.cpu(), 1.0, buckets, mul_prev, mul_cur)
        assert torch.equal(torch.cat(got[r]).double().cpu(), want), r
    assert int(prev[3]) == toks["a"][-1] and int(prev[1]) == toks["b"][-1] and int(prev[0]) == 0 == int(prev[2])
    prev[3].zero_()                                    # a new request in a's slot: its first token takes the last row
    ctx = _step_ctx([2], [3], _i32([0, 1]), _i32([4, 2]))
    resid = torch.zeros(2, d, device=DEV)
    ops.bigram_add(resid, table, prev, ctx, buckets, mul_prev, mul_cur, vocab)
    assert torch.equal(resid[0], table[buckets]) and torch.equal(resid[1], table[(4 * mul_prev + 2 * mul_cur) % buckets])


def _feed(steps, slots, rows, run):
    """Feed the requests' rows in the portions of ``steps`` ({request: count} per step); ``run(step rows, ctx)``
    returns one output row per input row.  Returns {request: all its output rows}."""
    at, got = {r: 0 for r in slots}, {r: [] for r in slots}
    for step in steps:
        lens = list(step.values())
        x = torch.cat([rows[r][at[r]:at[r] + k] for r, k in step.items()]).contiguous()
        y = run(x, _step_ctx(lens, [slots[r] for r in step]))
        o = 0
        for r, k in step.items():
            got[r].append(y[o:o + k])
            at[r] += k
            o += k
    return {r: torch.cat(v).double().cpu() for r, v in got.items()}


STEPS = [dict(a=5, b=1, c=2), dict(a=1, c=1), dict(b=11, a=2, c=1), dict(c=1), dict(c=9, a=1), dict(b=2, c=37)]


@pytest.mark.parametrize("Hh,dk,dv", [(3, 8, 12), (2, 20, 7), (1, 6, 40), (4, 64, 64), (2, 128, 33), (1, 256, 16),
                                      (8, 32, 128), (6, 16, 90)])
def test_lightning_attention_over_portions_and_reused_slots(ops, Hh, dk, dv):
    """Three requests in portions of unequal sizes (one left out of some steps) against the plain recurrence over each
    whole sequence, with the norm over all heads and the sigmoid gate; then a cleared slot is used again."""
    gen = torch.Generator(device=DEV).manual_seed(dk + dv)
    ld = 2 * Hh * dk + 2 * Hh * dv + 3
    k_off, v_off, g_off = Hh * dk + 1, 2 * Hh * dk + 2, 2 * Hh * dk + Hh * dv + 3
    decay = torch.tensor([0.5, 0.9, 0.99, 1.0, 0.999, 0.7, 0.8, 0.95][:Hh], device=DEV)
    norm_w = 1 + 0.3 * torch.randn(Hh * dv, device=DEV, generator=gen)
    state = torch.zeros(5, Hh * dv * dk, device=DEV)
    slots = {"a": 2, "b": 0, "c": 4}
    total = {r: sum(s.get(r, 0) for s in STEPS) for r in slots}
    proj = {r: torch.randn(total[r], ld, device=DEV, generator=gen) for r in slots}

    def run(x, ctx):
        o = ops.lightning_recurrence(x, 0, k_off, v_off, decay, state, ctx, Hh, dk, dv)
        return ops.gated_rmsnorm(o, x[:, g_off:g_off + Hh * dv], norm_w, 1e-4, 1, Hh * dv, torch.float32, "sigmoid")

    def plain(x):
        x = x.double().cpu()
        T = x.shape[0]
        q, k = P.silu(x[:, :Hh * dk]).view(T, Hh, dk), P.silu(x[:, k_off:k_off + Hh * dk]).view(T, Hh, dk)
        v = P.silu(x[:, v_off:v_off + Hh * dv]).view(T, Hh, dv)
        o = P.decaying_linear_attention(q, k, v, decay.double().cpu().tolist()).reshape(T, Hh * dv)
        return P.rms(o, 1e-4) * norm_w.double().cpu() * torch.sigmoid(x[:, g_off:g_off + Hh * dv])

    got = _feed(STEPS, slots, proj, run)
    for r in slots:
        want = plain(proj[r])
        assert (got[r] - want).abs().max() <= 2e-5 * max(1.0, want.abs().max().item()), r
    assert not state[1].any() and not state[3].any()             # the slots of no request were never written
    state[slots["a"]].zero_()
    fresh = {"a": torch.randn(7, ld, device=DEV, generator=gen)}
    again = _feed([dict(a=3), dict(a=4)], {"a": slots["a"]}, fresh, run)["a"]
    want = plain(fresh["a"])
    assert (again - want).abs().max() <= 2e-5 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,N,taps", [(24, 5, 3), (36, 40, 1), (128, 16, 4), (200, 24, 2), (40, 100, 5), (16, 256, 4)])
def test_selective_scan_over_portions_and_reused_slots(ops, inner, N, taps, out_dtype):
    gen = torch.Generator(device=DEV).manual_seed(inner + N)
    rnd = lambda *s: torch.randn(*s, device=DEV, generator=gen)
    conv, conv_b = rnd(inner, taps) * 0.7, rnd(inner) * 0.3
    a_log, d_skip, dt_b = rnd(inner, N) * 0.5, 1 + 0.2 * rnd(inner), rnd(inner) * 0.5
    tail_off = N * inner
    state = torch.zeros(5, tail_off + (taps - 1) * inner, device=DEV)
    slots = {"a": 2, "b": 0, "c": 4}
    total = {r: sum(s.get(r, 0) for s in STEPS) for r in slots}
    ld = 2 * inner + 1                         # rows of [x | z | dt | B | C]; dt, B, C stand for their products' results
    rows = {r: torch.cat([rnd(total[r], ld), rnd(total[r], inner) * 0.5, rnd(total[r], 2 * N)], dim=1) for r in slots}
    scale = 0.6

    def run(x, ctx):
        xz = x[:, :ld]
        xc, xr = ops.scan_conv(xz, conv, conv_b, state, tail_off, ctx, inner, taps, out_dtype)
        assert xr.dtype == out_dtype and (xr.float() - xc).abs().max() <= 1e-2 * xc.abs().max()
        both = torch.full((x.shape[0], inner + 5), float("nan"), device=DEV, dtype=out_dtype)
        ops.selective_scan(xz, xc, x[:, ld:ld + inner].contiguous(), x[:, ld + inner:], a_log, d_skip, dt_b, state,
                           tail_off, ctx, both[:, 5:], scale, inner, N, taps)
        assert torch.isnan(both[:, :5]).all()
        return both[:, 5:].float()

    def plain(x):
        x = x.double().cpu()
        xc = P.silu(P.causal_conv(x[:, :inner], conv.double().cpu(), conv_b.double().cpu()))
        dt = P.softplus(x[:, ld:ld + inner] + dt_b.double().cpu())
        y = P.diagonal_scan(xc, dt, -torch.exp(a_log.double().cpu()), x[:, ld + inner:ld + inner + N],
                            x[:, ld + inner + N:], d_skip.double().cpu())
        return y * P.silu(x[:, inner:2 * inner]) * scale

    tol = 2e-5 if out_dtype == torch.float32 else 1e-2
    got = _feed(STEPS, slots, rows, run)
    for r in slots:
        want = plain(rows[r])
        assert (got[r] - want).abs().max() <= tol * max(1.0, want.abs().max().item()), r
    assert not state[1].any() and not state[3].any()
    state[slots["a"]].zero_()
    fresh = {"a": torch.cat([rnd(7, ld), rnd(7, inner) * 0.5, rnd(7, 2 * N)], dim=1)}
    again = _feed([dict(a=1), dict(a=1), dict(a=5)], {"a": slots["a"]}, fresh, run)["a"]
    want = plain(fresh["a"])
    assert (again - want).abs().max() <= tol * max(1.0, want.abs().max().item())


def test_a_scan_with_a_long_memory_keeps_its_digits(ops):
    """Decays within 1e-3 to 1e-4 of 1 over 1,500 tokens, cut into portions: a float32 factor exp(dt A) keeps two or
    three digits of 1 - exp(dt A), and with it the read-outs end 4e-6 and more of their size away from the float64
    scan (measured with a correctly rounded exponential); moving the state by (exp(dt A) - 1) S + b stays below 1e-6.
    The bound lies between the two."""
    inner, N, taps, T = 48, 16, 2, 1500
    gen = torch.Generator(device=DEV).manual_seed(5)
    rnd = lambda *s: torch.randn(*s, device=DEV, generator=gen)
    conv, conv_b = rnd(inner, taps) * 0.7, rnd(inner) * 0.3
    a_log = torch.log(torch.full((inner, N), 0.01, device=DEV) * (1 + torch.arange(N, device=DEV)))   # A = -0.01 .. -0.16
    d_skip, dt_b = torch.zeros(inner, device=DEV), torch.full((inner,), -5.0, device=DEV)            # dt around 0.007
    tail_off = N * inner
    state = torch.zeros(2, tail_off + (taps - 1) * inner, device=DEV)
    ld = 2 * inner
    rows = {"a": torch.cat([rnd(T, ld), rnd(T, inner) * 0.5, rnd(T, 2 * N)], dim=1)}

    def run(x, ctx):
        xz = x[:, :ld]
        xc, _ = ops.scan_conv(xz, conv, conv_b, state, tail_off, ctx, inner, taps, torch.float32)
        y = torch.empty(x.shape[0], inner, device=DEV)
        ops.selective_scan(xz, xc, x[:, ld:ld + inner].contiguous(), x[:, ld + inner:], a_log, d_skip, dt_b, state,
                           tail_off, ctx, y, 1.0, inner, N, taps)
        return y

    steps = [dict(a=700), dict(a=1), dict(a=3), dict(a=500), dict(a=1), dict(a=295)]
    got = _feed(steps, {"a": 1}, rows, run)["a"]
    x = rows["a"].double().cpu()
    xc = P.silu(P.causal_conv(x[:, :inner], conv.double().cpu(), conv_b.double().cpu()))
    dt = P.softplus(x[:, ld:ld + inner] + dt_b.double().cpu())
    want = P.diagonal_scan(xc, dt, -torch.exp(a_log.double().cpu()), x[:, ld + inner:ld + inner + N],
                           x[:, ld + inner + N:], d_skip.double().cpu()) * P.silu(x[:, inner:2 * inner])
    assert (got - want).abs().max() <= 2e-6 * want.abs().max(), ((got - want).abs().max(), want.abs().max())


def _paged_keys(dtype, G, hd, vd, ps, q_lens, kv_lens, seed, values_are_keys):
    """Random keys (and values) of every request in pages handed out in scrambled order."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    ks = [torch.randn(L, G, hd, device=DEV, generator=g).to(dtype) for L in kv_lens]
    vs = ks if values_are_keys else [torch.randn(L, G, vd, device=DEV, generator=g).to(dtype) for L in kv_lens]
    pages_per = [-(-L // ps) for L in kv_lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(seed + 1))[:sum(pages_per)]
    entry = G * hd if values_are_keys else G * (hd + vd)
    cache = torch.randn(n_pages, ps * entry, device=DEV, generator=g).to(dtype)
    indptr = [0] + list(np.cumsum(pages_per))
    qo = [0] + list(np.cumsum(q_lens))
    pos = torch.cat([torch.arange(L - q, L) for q, L in zip(q_lens, kv_lens)]).to(DEV, torch.int32)
    ctx = _step_ctx(q_lens, [0] * len(q_lens), pos)
    ctx.max_q_len, ctx.max_kv_len, ctx.extras = max(q_lens), max(kv_lens), {"min_q_len": min(q_lens)}
    tables = SimpleNamespace(kv_indptr=_i32(indptr), kv_indices=perm.to(DEV, torch.int32), page_size=ps)

    def fill():
        for e, L in enumerate(kv_lens):
            for p in range(L):
                page = cache[int(perm[indptr[e] + p // ps])]
                page[:G * ps * hd].view(G, ps, hd)[:, p % ps] = ks[e][p]
                if not values_are_keys:
                    page[G * ps * hd:].view(G, ps, vd)[:, p % ps] = vs[e][p]
    return ks, vs, cache, ctx, tables, fill, qo


def _attention_case(ops, dtype, Hq, G, hd, vd, ps, q_lens, kv_lens, window=0, chunk=0, softcap=0.0, gated=False,
                    values_are_keys=False, sink=None, out_scale=1.0, spike=None, seed=0, scale=0.25, plain_part=False):
    ks, vs, cache, ctx, tables, fill, qo = _paged_keys(dtype, G, hd, vd, ps, q_lens, kv_lens, seed, values_are_keys)
    g = torch.Generator(device=DEV).manual_seed(seed + 5)
    n = sum(q_lens)
    q = torch.randn(n, Hq, hd, device=DEV, generator=g)
    if spike is not None:                  # one key whose score with the last query of a request stands out
        e, key, head = spike
        t = qo[e] + q_lens[e] - 1
        q[t, head] = 0
        q[t, head, hd - 1] = 40.0
        ks[e][:, :, hd - 1] = ks[e][:, :, hd - 1].clamp(-1, 1)
        ks[e][key, head // (Hq // G), hd - 1] = 30.0
    q = q.to(dtype)
    fill()
    gate = torch.randn(n, Hq * vd + 3, device=DEV, generator=g)[:, 3:] if gated else None
    both = torch.full((n, Hq * vd + 7), float("nan"), device=DEV, dtype=dtype)
    if plain_part:       # the plain attention part's kernels (tensor cores in bfloat16), which need vd == hd
        ctx.kv_len = _i32(kv_lens)
        heads = torch.full((n, Hq * vd), float("nan"), device=DEV, dtype=dtype)
        ops.paged_attention(q.view(n, Hq * hd), heads, cache.view(cache.shape[0], 2, -1), ctx, tables, Hq, G, hd, scale,
                            window, chunk, sink, ops.sink_table(sink) if sink is not None else None, softcap)
        ops.gate_mul(heads, gate, both[:, :Hq * vd], out_scale)
        ops.check_status()
    else:
        ops.masked_attention(q.view(n, Hq * hd), both[:, :Hq * vd], cache, ctx, tables, Hq, G, hd, vd, scale, window,
                             chunk, sink, softcap, values_are_keys, gate, out_scale)
    torch.cuda.synchronize()
    assert torch.isnan(both[:, Hq * vd:]).all()
    want = torch.empty(n, Hq, vd, dtype=F64)
    for e, (ql, L) in enumerate(zip(q_lens, kv_lens)):
        if window:
            visible = lambda i, j: i - j < window
        elif chunk:
            visible = lambda i, j: i // chunk == j // chunk
        else:
            visible = lambda i, j: True
        qq = torch.cat([torch.zeros(L - ql, Hq, hd, dtype=F64), q[qo[e]:qo[e + 1]].double().cpu()])
        full = P.softmax_attention(qq, ks[e].double().cpu(), vs[e].double().cpu(), scale, visible, softcap,
                                   sink_one=sink is not None)
        want[qo[e]:qo[e + 1]] = full[L - ql:]
    if gated:
        want = want * torch.sigmoid(gate.double().cpu()).view(n, Hq, vd)
    return both[:, :Hq * vd].double().cpu().view(n, Hq, vd), want * out_scale, vs


WINDOW_SHAPES = [  # Hq, G, hd, vd, page, window, q_lens, kv_lens
    (4, 2, 12, 20, 4, 10, [1, 5, 1], [37, 5, 9]),
    (6, 1, 48, 96, 16, 96, [1, 1, 40], [300, 96, 140]),
    (3, 3, 16, 8, 3, 7, [2, 9], [9, 30]),
    (8, 2, 64, 32, 16, 128, [1, 130], [1000, 400]),
    (2, 2, 256, 256, 8, 33, [1, 3], [70, 33]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", WINDOW_SHAPES, ids=lambda s: f"H{s[0]}G{s[1]}d{s[2]}v{s[3]}ps{s[4]}w{s[5]}")
def test_window_attention_with_soft_cap_and_gate(ops, dtype, shape):
    Hq, G, hd, vd, ps, window, q_lens, kv_lens = shape
    for softcap, gated, out_scale in ((0.0, False, 1.0), (3.0, True, 0.6)):
        got, want, _ = _attention_case(ops, dtype, Hq, G, hd, vd, ps, q_lens, kv_lens, window=window, softcap=softcap,
                                       gated=gated, out_scale=out_scale, seed=hd, scale=0.5)
        assert (got - want).abs().max() <= _tol(dtype) * max(1.0, want.abs().max().item())


TENSOR_CORE_SHAPES = [  # Hq, G, hd, page, window, q_lens, kv_lens: split keys, 64-row and 128-row prompt kernels
    (8, 2, 64, 16, 128, [1, 1, 1], [1000, 37, 128]),
    (16, 4, 128, 16, 1024, [1, 300], [2500, 1500]),
    (4, 4, 64, 8, 100, [70, 1, 5], [333, 90, 105]),
    (6, 1, 256, 32, 96, [1, 40], [300, 140]),
]


@pytest.mark.parametrize("shape", TENSOR_CORE_SHAPES, ids=lambda s: f"H{s[0]}G{s[1]}d{s[2]}ps{s[3]}w{s[4]}")
def test_window_soft_cap_and_gate_on_the_tensor_core_kernels(ops, shape):
    Hq, G, hd, ps, window, q_lens, kv_lens = shape
    for softcap, gated, out_scale in ((0.0, False, 1.0), (3.0, True, 0.6), (30.0, False, 1.0)):
        got, want, _ = _attention_case(ops, torch.bfloat16, Hq, G, hd, hd, ps, q_lens, kv_lens, window=window,
                                       softcap=softcap, gated=gated, out_scale=out_scale, seed=hd, scale=0.5,
                                       plain_part=True)
        assert (got - want).abs().max() <= 2e-2 * max(1.0, want.abs().max().item()), (softcap, gated)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("back", [0, 1, 95, 96, 97, 111, 112, 200, 299])
def test_one_key_decides_inside_the_window_on_the_tensor_core_kernels(ops, hd, back):
    for q_lens in ([1], [7], [150]):
        L = 300
        got, want, vs = _attention_case(ops, torch.bfloat16, 8, 2, hd, hd, 16, q_lens, [L], window=96, softcap=50.0,
                                        spike=(0, L - 1 - back, 4), seed=back, plain_part=True)
        assert (got - want).abs().max() <= 2e-2 * max(1.0, want.abs().max().item())
        hit = (got[-1, 4] - vs[0][L - 1 - back, 1].double().cpu()).abs().max() <= 5e-2
        assert hit == (back < 96), (back, q_lens)


def test_the_soft_cap_bounds_a_score_that_would_take_all_the_weight(ops):
    """One score of 300 among scores near 0: without the cap its key has all the weight, with a cap of 2 it has
    e^2 / (e^2 + others)."""
    got, want, vs = _attention_case(ops, torch.float32, 2, 1, 16, 16, 8, [1], [40], softcap=2.0, spike=(0, 17, 1), seed=3)
    assert (got - want).abs().max() <= 2e-5 * want.abs().max()
    assert (got[0, 1] - vs[0][17, 0].double().cpu()).abs().max() > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("back", [0, 1, 95, 96, 97, 111, 112, 200, 299])
def test_one_key_decides_inside_the_window_and_is_unseen_outside(ops, dtype, back):
    """A window of 96 over 300 keys in pages of 16: the key ``back`` positions before the query gets a score that
    stands out.  Inside the window the output is that key's value; outside, the key changes nothing.  From a decoded
    token and from the end of a portion."""
    for q_lens in ([1], [7]):
        L = 300
        got, want, vs = _attention_case(ops, dtype, 6, 1, 48, 96, 16, q_lens, [L], window=96, spike=(0, L - 1 - back, 4),
                                        seed=back)
        assert (got - want).abs().max() <= _tol(dtype) * max(1.0, want.abs().max().item())
        hit = (got[-1, 4] - vs[0][L - 1 - back, 0].double().cpu()).abs().max() <= 2e-2
        assert hit == (back < 96), (back, q_lens)


CHUNK_SHAPES = [  # Hq, G, hd, page, chunk, q_lens, kv_lens
    (3, 3, 16, 4, 12, [1, 5, 1], [37, 5, 12]),
    (6, 2, 64, 16, 64, [1, 1, 70], [300, 64, 140]),
    (2, 1, 6, 3, 7, [2, 9], [9, 30]),
    (8, 4, 128, 8, 100, [1, 130], [1000, 400]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", CHUNK_SHAPES, ids=lambda s: f"H{s[0]}G{s[1]}d{s[2]}ps{s[3]}c{s[4]}")
def test_chunk_attention_over_its_own_keys_with_one_in_the_denominator(ops, dtype, shape):
    Hq, G, hd, ps, chunk, q_lens, kv_lens = shape
    sink = torch.zeros(Hq, device=DEV)
    got, want, _ = _attention_case(ops, dtype, Hq, G, hd, hd, ps, q_lens, kv_lens, chunk=chunk, values_are_keys=True,
                                   sink=sink, seed=hd)
    assert (got - want).abs().max() <= _tol(dtype) * max(1.0, want.abs().max().item())


def test_the_added_one_shows_when_every_score_is_small(ops):
    """All scores 0 over 20 keys: with the added one every key gets 1/21 instead of 1/20."""
    sink = torch.zeros(2, device=DEV)
    got, want, _ = _attention_case(ops, torch.float32, 2, 1, 16, 16, 8, [1], [20], values_are_keys=True, sink=sink,
                                   seed=1, scale=0.0)
    assert (got - want).abs().max() <= 2e-5
    _, plain_mean, _ = _attention_case(ops, torch.float32, 2, 1, 16, 16, 8, [1], [20], values_are_keys=True, seed=1,
                                       scale=0.0)
    assert torch.allclose(want * 21 / 20, plain_mean, atol=1e-9)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key", [0, 255, 256, 257, 271, 272, 319, 320, 321, 350, 399])
def test_one_key_decides_inside_its_chunk_and_is_unseen_outside(ops, dtype, key):
    """Chunks of 64 over 400 keys in pages of 16, the query at position 399 (chunk 384..399) or 330 (chunk 320..383)."""
    for L, first in ((400, 384), (331, 320)):
        if key >= L:
            continue
        for q_lens in ([1], [min(9, L)]):
            sink = torch.zeros(6, device=DEV)
            got, want, vs = _attention_case(ops, dtype, 6, 2, 64, 64, 16, q_lens, [L], chunk=64, values_are_keys=True,
                                            sink=sink, spike=(0, key, 5), seed=key)
            assert (got - want).abs().max() <= _tol(dtype) * max(1.0, want.abs().max().item())
            hit = (got[-1, 5] - vs[0][key, 1].double().cpu()).abs().max() <= 0.3
            assert hit == (key >= first), (key, L, q_lens)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,G,hd,vd,rot,ps", [(4, 2, 12, 20, 8, 4), (6, 1, 48, 96, 48, 16), (3, 3, 16, 0, 0, 8),
                                                (8, 2, 64, 32, 64, 16)])
def test_interleaved_rotation_and_append_from_wider_rows(ops, dtype, Hq, G, hd, vd, rot, ps):
    """q/k/v preparation from the leading columns of wider rows, rotation of adjacent pairs of the first ``rot``
    numbers, and (vd 0) pages of keys alone; positions far out, scrambled pages, nothing else written."""
    gen = torch.Generator(device=DEV).manual_seed(hd + vd)
    n = 6
    width = (Hq + G) * hd + G * vd
    rows = torch.randn(n, width + 4 * Hq, device=DEV, generator=gen)
    positions = [0, 1, ps - 1, ps, 4001, 70001]
    n_pages = 70001 // ps + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    entry = G * (hd + vd)
    cache = torch.zeros(n_pages, ps * entry, device=DEV, dtype=dtype)
    base = 50000.0
    freqs = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F64) if rot else None
    table = ops.rope_frequency_table(freqs, DEV) if rot else None
    q = ops.qkv_prepare(rows[:, :width], Hq, G, hd, vd, None, table, rot, True, 1.0, 0.0, _i32(positions),
                        _i32([0] * n), _i32([0, n_pages]), perm.to(DEV), cache, ps)
    x = rows.double().cpu()
    qw = x[:, :Hq * hd].view(n, Hq, hd).clone()
    kw = x[:, Hq * hd:(Hq + G) * hd].view(n, G, hd).clone()
    for t, p in enumerate(positions):
        for i in range(rot // 2):
            a = p * base ** (-2.0 * i / rot)
            c, s = np.cos(a), np.sin(a)
            for w in (qw, kw):
                u, v = w[t, :, 2 * i].clone(), w[t, :, 2 * i + 1].clone()
                w[t, :, 2 * i], w[t, :, 2 * i + 1] = u * c - v * s, v * c + u * s
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (q.double().cpu().view(n, Hq, hd) - qw).abs().max() <= tol * qw.abs().max()
    touched = torch.zeros(n_pages, dtype=torch.bool)
    for t, p in enumerate(positions):
        page = cache[int(perm[p // ps])].double().cpu()
        touched[int(perm[p // ps])] = True
        assert (page[:G * ps * hd].view(G, ps, hd)[:, p % ps] - kw[t]).abs().max() <= tol * kw.abs().max()
        if vd:
            vw = x[t, (Hq + G) * hd:width].view(G, vd)
            assert (page[G * ps * hd:].view(G, ps, vd)[:, p % ps] - vw).abs().max() <= tol * vw.abs().max()
    assert not cache[~touched.to(DEV)].any()
    assert int((cache != 0).sum()) <= n * entry


# ------------------------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
@pytest.mark.parametrize("name", ["A", "B"])
def test_token_by_token_from_the_first_token(tmp_path, name, dtype):
    """A whole request decoded one token at a time (the first tokens of a sequence, every page border, window and
    chunk edge, the convolution's first inputs, long decoding) against the oracle."""
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    toks = H.random_tokens(150, cfg["vocab"], 4)
    eng = _engine(folder, dtype, page, 40)
    got = H.run_steps_in_process(eng, H.portions("t", toks, [1]))
    _compare(got, folder, {"t": toks}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_requests_reuse_pages_and_slots(tmp_path, name, dtype):
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    base = _requests(name)
    reqs = dict(base)
    for i, (rid, toks) in enumerate(base.items()):          # twice as many requests as there are slots
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
def test_a_model_of_recurrent_layers_alone_needs_no_pages(tmp_path, dtype):
    cfg, seed, page = CONFIGS["STATE"]
    folder = _folder(tmp_path, "STATE", dtype)
    reqs = {f"q{i}": H.random_tokens(n, cfg["vocab"], 7 + i) for i, n in enumerate([1, 5, 30, 77, 12, 3])}
    eng = _engine(folder, dtype, page, 1, max_requests=3)
    assert not eng.cache.groups and sum(s is not None for s in eng.cache.state_tensors) == 4    # three runs + last token
    got = H.run_steps_in_process(eng, H.mixed(reqs, seed=5, max_live=3))          # six requests through three slots
    _compare(got, folder, reqs, dtype)
    one = H.run_steps_in_process(eng, H.portions("q3", reqs["q3"], [2, 1, 9]))
    _rows_agree(one, {k: got[k] for k in one}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tmp_path, dtype):
    cfg, seed, page = CONFIGS["B"]
    folder = _folder(tmp_path, "B", dtype)
    reqs = _requests("B")
    steps = H.mixed(reqs, seed=3, max_live=4)
    got = H.run_trace_subprocess(folder, dtype, steps, tmp_path / "out", H.max_live_tokens(steps, round_to=64))
    _compare(got, folder, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,edge", [("WINDOW", "window"), ("CHUNK", "chunk")])
def test_a_token_outside_the_mask_is_unseen_and_the_first_inside_is_seen(tmp_path, name, edge, dtype):
    """One layer, a mask of 12 positions, no bigram rows (and the scan's branch multiplied by 0): changing a token
    that the mask hides from the positions 36..47 changes none of their logits, bit for bit; changing the first token
    they see changes them.  As one prompt, token by token, and in portions that cross the edge inside a page."""
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype, std=0.3)
    base = H.random_tokens(48, cfg["vocab"], 2)
    eng = _engine(folder, dtype, page, 12)
    # window: position 47 sees 36..47, position 36 sees 25..36; chunk: 36..47 see 36.. only
    cases = ((24, [], range(36, 48)), (25, [36], range(37, 48)), (35, range(36, 47), [47]), (0, [], range(36, 48))) \
        if edge == "window" else ((35, [], range(36, 48)), (36, range(36, 48), []), (23, [], range(36, 48)))
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
def test_a_far_token_decides_the_logits_through_the_state(tmp_path, dtype):
    """Changing ONE token far back (the first, one at a page border, one deep inside) changes the last position's
    logits in the oracle although every window and chunk has long passed it: the recurrent states carry it.  The
    engine follows, decoded alone and as the end of a portion."""
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
            assert err <= H.TOL[dtype], (where, err)
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
        eng.setup_caches(max_batch_size=3, max_seq_length=96, page_size=page, prefill_chunk_size=16, num_pages=50)
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
