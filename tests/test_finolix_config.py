"""The Finolix design without a GPU: its configuration reader, the order of its layer runs, its model description
against the tensors a folder holds, what its runs ask of the cache manager, and the plain implementation's own
mechanisms against closed forms."""
import math

import pytest
import torch

import plain_finolix as P
from batchspec_b200.config import ConfigError, config_from_json_dict
from batchspec_b200.models import get_model
from batchspec_b200.parts.base import Runtime


def latent(window=10, mlp="dense", scaling=True):
    rot = dict(base=5000.0, dims=4)
    if scaling:
        rot["scaling"] = dict(factor=4.0, original=32, fast=8.0, slow=1.0)
    m = dict(heads=3, dim=8, rot_dim=4, vdim=12, q_rank=20, kv_rank=24, scale=0.3, rot=rot)
    if window:
        m["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=m, mlp=dict(kind="dense", ff=40) if mlp == "dense" else mlp)


def attention(mlp=None):
    return dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.25,
                                             rot=dict(base=3000.0, dims=8)),
                mlp=mlp or dict(kind="moe", expert=dict(ff=16), router=dict(experts=5, top=2)))


def config(layers, streams=3, **kw):
    d = dict(architecture="Finolix", vocab=200, width=48, norm=dict(eps=1e-5), layers=layers)
    if streams:
        d["streams"] = streams
    d.update(kw)
    return d


def model(d):
    return get_model(config_from_json_dict(d), Runtime(torch.float32, torch.device("cpu")))


def test_reader_takes_every_size_from_the_file_and_round_trips():
    layers = [latent(), attention(), latent(window=None, mlp=None)]
    d = config(layers + [dict(layers[1], weights_of=1), dict(layers[0], weights_of=0)])
    cfg = config_from_json_dict(d)
    assert (cfg.vocab_size, cfg.width, cfg.norm_eps, cfg.streams) == (200, 48, 1e-5, 3) and not cfg.unread_keys
    assert cfg.run_order() == [0, 1, 2, 1, 0]
    assert config_from_json_dict(cfg.to_json_dict()) == cfg
    d2 = config([latent()], foo=1)
    d2["layers"][0]["mixer"]["bar"] = 2
    assert set(config_from_json_dict(d2).unread_keys) == {"foo", "layers[0].mixer.bar"}
    assert config_from_json_dict(config([latent()], streams=None)).streams == 0


@pytest.mark.parametrize("break_it", [
    lambda d: d["layers"][0].update(type="conv"), lambda d: d["layers"][0]["mixer"].update(rot_dim=6),
    lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3), lambda d: d["layers"][0]["mixer"]["mask"].update(size=0),
    lambda d: d["layers"][1]["mixer"].update(heads=4, kv_heads=3), lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14),
    lambda d: d["layers"][1]["mlp"]["router"].update(top=6), lambda d: d["layers"][1]["mlp"].update(kind="glu"),
    lambda d: d.update(streams=0), lambda d: d.update(streams=17), lambda d: d["layers"][2].update(weights_of=2),
    lambda d: d["layers"][2].update(weights_of=1), lambda d: d["norm"].update(eps=0.0),
    lambda d: d["layers"][2].update(weights_of=5),
])
def test_reader_refuses_what_cannot_be_run(break_it):
    layers = [latent(), attention()]
    d = config(layers + [dict(layers[0], weights_of=0)])
    config_from_json_dict(d)
    break_it(d)
    with pytest.raises(ConfigError):
        config_from_json_dict(d)


def test_tensor_names_block_kinds_and_runs():
    layers = [latent(), attention(), latent(window=None, mlp=None)]
    m = model(config(layers + [dict(layers[1], weights_of=1)]))
    names = set(m.param_specs())
    assert {"embed", "head", "final.norm", "l0.mix.dq.norm", "l0.mix.sink", "l0.hc1.mix", "l0.hc2.in", "l0.ls2",
            "l0.mlp.up", "l1.mix.q.norm", "l1.mix.g", "l1.mlp.router.b", "l1.mlp.e4.gate", "l2.hc1.out"} <= names
    assert not any(n.startswith(("l3.", "l2.mlp", "l2.hc2", "l2.norm2")) for n in names)
    assert m.param_specs()["l1.mix.g"].shape == (4, 48) and m.param_specs()["l0.hc1.mix"].shape == (3, 3)
    assert [b.kind for b in m.blocks] == ["hyper_prenorm", "hyper_prenorm", "hyper_prenorm_mixer"]
    assert [r.layer for r in m.spec.order] == [0, 1, 2, 1] and m.spec.streams == 3
    needs = m.cache_needs()
    assert [(n.cache.policy, n.cache.window, n.cache.tensors) for n in needs] == \
        [("window", 10, 1), ("full", None, 1), ("full", None, 1), ("full", None, 1)]
    assert needs[0].cache.entry_shape == (28,) and all(n.state is None for n in needs)
    one = model(config(layers, streams=None))
    assert [b.kind for b in one.blocks] == ["prenorm_scaled", "prenorm_scaled", "prenorm_mixer_scaled"]
    assert not any(".hc" in n for n in one.param_specs()) and one.spec.streams == 0


def test_plain_rotation_pairs_and_yarn():
    f, mag = P.yarn_frequencies(100.0, 4, None)
    assert mag == 1.0 and f == [1.0, 100.0 ** -0.5]
    x = torch.zeros(1, 1, 6, dtype=P.F)
    x[0, 0, 0] = 1.0
    by_pairs = P.rotate(x, [1], [math.pi / 2, 0.0], 1.0, True)
    by_halves = P.rotate(x, [1], [math.pi / 2, 0.0], 1.0, False)
    assert abs(by_pairs[0, 0, 1] - 1.0) < 1e-12 and abs(by_halves[0, 0, 2] - 1.0) < 1e-12
    assert by_pairs[0, 0, 4:].abs().max() == 0
    f2, mag2 = P.yarn_frequencies(10000.0, 8, dict(factor=4.0, original=64, fast=1e9, slow=1e-9))
    base = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert abs(mag2 - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert f2[0] == base[0] and abs(f2[-1] - base[-1] * (3 / 7 / 4.0 + 4 / 7)) < 1e-15      # ramp from index 0 to 7


def test_plain_sink_window_and_routing():
    q = torch.zeros(4, 1, 2, dtype=P.F)
    k = torch.zeros(4, 1, 2, dtype=P.F)
    v = torch.arange(4, dtype=P.F).reshape(4, 1, 1)
    out = P.softmax_attention(q, k, v, 1.0, window=2, sink=torch.tensor([math.log(2.0)], dtype=P.F))
    assert torch.allclose(out.flatten(), torch.tensor([0.0, 0.25, 0.75, 1.25], dtype=P.F))
    idx, wt = P.route(torch.eye(3, dtype=P.F), torch.tensor([[1.0, 0, 0], [0, 2.0, 0], [0, 0, 3.0]]),
                      torch.tensor([0.0, 0.0, -10.0]), 2)
    assert idx[2].tolist() == [0, 1] and torch.allclose(wt[0], torch.softmax(torch.tensor([1.0, 0.0], dtype=P.F), 0))


def test_plain_streams_reduce_to_a_residual_sum():
    """With one stream, in = out = mix = 1, the streams are the ordinary residual sum."""
    torch.manual_seed(0)
    d = config([latent(mlp="dense")], streams=1)
    m = model(d)
    w = {n: 0.2 * torch.randn(ps.shape) for n, ps in m.param_specs().items()}
    for q in (1, 2):
        for n in ("in", "out", "mix"):
            w[f"l0.hc{q}.{n}"] = torch.ones_like(w[f"l0.hc{q}.{n}"])
    toks = [3, 9, 150, 7, 7, 21]
    a, _ = P.forward(d, w, toks)
    b, _ = P.forward(config([latent(mlp="dense")], streams=None), w, toks)
    assert torch.allclose(a, b, atol=1e-12)
