"""The Tokolorn design without a GPU: its configuration reader, the order of its layer runs, its model description
against the tensors a folder holds, what its runs ask of the cache manager, and the plain implementation's own
mechanisms against closed forms."""
import math

import pytest
import torch

import plain_tokolorn as P
from batchspec_b200.cache.manager import CacheManager
from batchspec_b200.config import ConfigError, config_from_json_dict, get_config
from batchspec_b200.models import get_model
from batchspec_b200.parts.base import Runtime


def lightning(heads=3, dim=8, vdim=12, decay=(0.5, 0.9, 0.99), mlp="dense"):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)),
                mlp=dict(kind="dense", ff=40) if mlp == "dense" else mlp)


def parallel(mlp=None):
    left = dict(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.3, softcap=5.0, mask=dict(size=10),
                rot=dict(base=5000.0, dims=8))
    return dict(type="parallel", mixer=dict(left=left, right=dict(inner=24, state=5, dt_rank=3, conv=3), left_scale=0.6,
                                            right_scale=0.5), mlp=mlp)


def attention(heads=3, kv_heads=3, dim=16, size=12):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=0.25,
                                             mask=dict(size=size)), mlp=dict(kind="dense", ff=56))


def config(layers, loop=None, **kw):
    d = dict(architecture="Tokolorn", vocab=200, width=48, norm=dict(eps=1e-5), logit_scale=0.7,
             embedding=dict(scale=3.0, bigram=dict(buckets=61, mul_prev=5, mul_cur=3)), layers=layers)
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    d.update(kw)
    return d


def test_reader_takes_every_size_from_the_file_and_round_trips():
    d = config([lightning(), parallel(), attention()], loop=(0, 2, 3))
    cfg = config_from_json_dict(d)
    assert (cfg.vocab_size, cfg.width, cfg.norm_eps, cfg.logit_scale, cfg.embed_scale) == (200, 48, 1e-5, 0.7, 3.0)
    assert cfg.bigram == dict(buckets=61, mul_prev=5, mul_cur=3)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (0, 2, 3) and not cfg.unread_keys
    assert config_from_json_dict(cfg.to_json_dict()) == cfg
    d2 = config([lightning()], foo=1)
    d2["layers"][0]["mixer"]["bar"] = 2
    assert set(config_from_json_dict(d2).unread_keys) == {"foo", "layers[0].mixer.bar"}
    plain = config_from_json_dict(config([attention()], embedding=dict(scale=2.0)))
    assert plain.bigram is None and get_model(plain, Runtime(torch.float32, torch.device("cpu"))).input_part is None


@pytest.mark.parametrize("break_it", [
    lambda d: d["layers"][0].update(type="conv"), lambda d: d["layers"][0]["mixer"].update(decay=[0.5, 0.9]),
    lambda d: d["layers"][1]["mixer"]["left"].update(heads=4, kv_heads=3),
    lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
    lambda d: d["layers"][1]["mixer"]["left"]["mask"].update(size=0),
    lambda d: d["layers"][1]["mixer"]["right"].update(conv=0), lambda d: d["layers"][1]["mixer"].pop("left_scale"),
    lambda d: d["layers"][2]["mixer"].update(vdim=8), lambda d: d.update(loop=dict(start=1, stop=5, times=2)),
    lambda d: d["layers"][0]["mlp"].update(kind="moe"), lambda d: d["norm"].update(eps=0.0),
    lambda d: d["embedding"]["bigram"].update(buckets=0), lambda d: d["layers"][2]["mixer"].pop("scale")])
def test_reader_refuses_what_the_engine_cannot_run(break_it):
    d = config([lightning(), parallel(), attention()])
    break_it(d)
    with pytest.raises(ConfigError):
        config_from_json_dict(d)


def test_run_order_and_the_plain_order_agree():
    for loop, want in (((0, 2, 3), [0, 1, 0, 1, 0, 1, 2]), ((1, 3, 2), [0, 1, 2, 1, 2]), ((1, 1, 4), [0, 1, 2]),
                       ((0, 3, 1), [0, 1, 2]), (None, [0, 1, 2])):
        d = config([lightning(), parallel(), attention()], loop=loop)
        assert config_from_json_dict(d).run_order() == want == P.run_order(d)


def test_tensor_names_cache_needs_and_state():
    d = config([lightning(), parallel(), attention(), lightning(mlp=None)], loop=(0, 2, 2))
    model = get_model(config_from_json_dict(d), Runtime(torch.bfloat16, torch.device("cpu")))
    specs = {k: tuple(v.shape) for k, v in model.param_specs().items()}
    assert specs["embed"] == (200, 48) and specs["bigram"] == (62, 48) and specs["head"] == (200, 48)
    assert specs["final.norm"] == () and specs["l0.norm1"] == () and specs["l0.ls2"] == (48,)
    assert specs["l0.mix.q"] == (24, 48) and specs["l0.mix.v"] == (36, 48) and specs["l0.mix.norm"] == (36,)
    assert specs["l1.mix.left.k"] == (24, 48) and specs["l1.mix.left.g"] == (80, 48) and specs["l1.mix.left.o"] == (48, 80)
    assert specs["l1.mix.right.in"] == (48, 48) and specs["l1.mix.right.x"] == (13, 24) and specs["l1.mix.right.dt"] == (24, 3)
    assert specs["l1.mix.right.conv"] == (24, 3) and specs["l1.mix.right.conv.b"] == (24,) and specs["l1.mix.right.A_log"] == (24, 5)
    assert "l1.mlp.gate" not in specs and "l1.norm2" not in specs and "l2.mix.v" not in specs and "l3.ls2" not in specs
    needs = model.cache_needs()
    assert len(needs) == 7                                   # six layer runs and the input part's last token
    assert [n.cache.policy if n.cache else None for n in needs] == [None, "window", None, "window", "chunk", None, None]
    assert needs[1].cache.window == 10 and needs[1].cache.entry_shape == (2 * (12 + 20),) and needs[1].cache.tensors == 1
    assert needs[4].cache.window == 12 and needs[4].cache.entry_shape == (3 * 16,) and needs[4].cache.tensors == 1
    assert needs[0].state.shape == (3 * 12 * 8,) and needs[1].state.shape == (5 * 24 + 2 * 24,)
    assert needs[6].state.dtype == torch.int32 and needs[6].cache is None
    assert model.graph_safe
    cache = CacheManager(needs, 4, 16, 3, torch.bfloat16, "cpu", allocate=False)
    assert len(cache.groups) == 2 and len(cache.layer_caches) == 7
    rc = cache.admit("a")
    cache.reserve("a", 30)
    cache.commit("a", 30)
    assert [p >= 0 for p in rc.tables[0]] == [False] * 5 + [True] * 3        # the window of 10 keeps positions 21..
    assert [p >= 0 for p in rc.tables[1]] == [False] * 6 + [True] * 2        # the chunk of 12 that holds position 30 starts at 24


def test_a_preset_by_name_builds():
    cfg = get_config("tiny-tokolorn")
    model = get_model(cfg, Runtime(torch.float32, torch.device("cpu")))
    assert cfg.architecture == "Tokolorn" and len(model.cache_needs()) == len(cfg.run_order()) + 1


def test_plain_mechanisms_against_closed_forms():
    F = torch.float64
    # a constant input under decay d: S_t = (1 + d + ... + d^t) k v^T, so o_t = (k . q) v (1 - d^(t+1)) / (1 - d)
    q, k, v = torch.tensor([1.0, 2.0], dtype=F), torch.tensor([0.5, -1.0], dtype=F), torch.tensor([3.0, 1.0, -2.0], dtype=F)
    T, d = 6, 0.8
    o = P.decaying_linear_attention(q.expand(T, 1, 2), k.expand(T, 1, 2), v.expand(T, 1, 3), [d])
    for t in range(T):
        assert torch.allclose(o[t, 0], (k @ q) * v * (1 - d ** (t + 1)) / (1 - d))
    # one channel, one state, constant step: S_t = a S_(t-1) + dt x B with a = exp(dt A)
    x, dt = torch.ones(5, 1, dtype=F), torch.full((5, 1), 0.5, dtype=F)
    y = P.diagonal_scan(x, dt, torch.tensor([[-2.0]], dtype=F), torch.full((5, 1), 3.0, dtype=F),
                        torch.full((5, 1), 2.0, dtype=F), torch.tensor([0.25], dtype=F))
    a, s = math.exp(-1.0), 0.0
    for t in range(5):
        s = a * s + 0.5 * 3.0
        assert abs(float(y[t, 0]) - (2.0 * s + 0.25)) < 1e-12
    # the last tap multiplies the token's own input; inputs before the start are zero
    c = P.causal_conv(torch.tensor([[1.0], [2.0], [4.0]], dtype=F), torch.tensor([[100.0, 10.0, 1.0]], dtype=F),
                      torch.tensor([0.5], dtype=F))
    assert c.flatten().tolist() == [1.5, 12.5, 124.5]
    # a window of 2 over equal scores: the mean of the last two values; with one in the denominator a third less
    qq, kk = torch.zeros(3, 1, 2, dtype=F), torch.zeros(3, 1, 2, dtype=F)
    vv = torch.tensor([[[1.0]], [[3.0]], [[7.0]]], dtype=F)
    w = P.softmax_attention(qq, kk, vv, 1.0, lambda i, j: i - j < 2)
    assert w.flatten().tolist() == [1.0, 2.0, 5.0]
    w1 = P.softmax_attention(qq, kk, vv, 1.0, lambda i, j: i // 2 == j // 2, sink_one=True)
    assert torch.allclose(w1.flatten(), torch.tensor([0.5, 4.0 / 3.0, 3.5], dtype=F))
    # the soft cap: c tanh(s / c) -> weights e^c' against 1
    s = P.softmax_attention(torch.tensor([[[10.0]], [[10.0]]], dtype=F), torch.tensor([[[0.0]], [[10.0]]], dtype=F),
                            torch.tensor([[[0.0]], [[1.0]]], dtype=F), 1.0, lambda i, j: True, softcap=2.0)
    e = math.exp(2.0 * math.tanh(50.0))
    assert abs(float(s[1, 0, 0]) - e / (e + 1.0)) < 1e-12
    # rotation of adjacent pairs keeps lengths, leaves the unrotated part, and turns position p by p * f
    x = torch.randn(4, 2, 6, dtype=F)
    r = P.rotate_interleaved(x, 100.0, 4)
    assert torch.allclose(r[..., 4:], x[..., 4:]) and torch.allclose(r[..., :4].norm(dim=-1), x[..., :4].norm(dim=-1))
    assert torch.allclose(r[0], x[0])
    assert torch.allclose(r[3, :, 2], x[3, :, 2] * math.cos(3 * 0.1) - x[3, :, 3] * math.sin(3 * 0.1))
    # the bigram row of the first token is the table's last
    rows = P.embed_rows([4, 2], torch.zeros(5, 3, dtype=F), torch.arange(24, dtype=F).view(8, 3), 1.0, 7, 5, 3)
    assert rows[0].tolist() == [21.0, 22.0, 23.0] and rows[1].tolist() == [15.0, 16.0, 17.0]       # (4*5 + 2*3) % 7 = 5
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=F))) - 0.8411919906082768) < 1e-12
