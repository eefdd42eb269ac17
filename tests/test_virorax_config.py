"""Virorax without a GPU: configuration, spec and manifest, refusals, and the plain
implementation's own properties."""
import copy
import math

import pytest
import torch

import plain_virorax as plain
import virorax_tiny as tiny
from cretif_b200.config import (ConfigError, build_virorax_spec, virorax_config_from_dict,
                                resolve_architecture)
from cretif_b200.engine.model import manifest


def _spec(cfg):
    return build_virorax_spec(virorax_config_from_dict(cfg))


def test_registered_and_parsed():
    assert resolve_architecture("Virorax").config_from_dict is virorax_config_from_dict
    cfg = virorax_config_from_dict(tiny.V_A)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.residual_mult, cfg.logit_softcap) == \
        (96, 64, 1e-5, 0.5, 8.0)
    assert cfg.loop == {"start": 1, "stop": 3, "times": 3}
    assert virorax_config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_schedule_of_a_repeated_span():
    spec = _spec(tiny.V_A)
    spec.validate()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.add_input for e in spec.schedule] == [False, False, False, True, False, True,
                                                    False, False]
    assert all(e.cache is None for e in spec.schedule)       # every run has its own cache
    spec = _spec(tiny.V_B)                                     # the span starts at layer 0
    assert [(e.layer, e.add_input) for e in spec.schedule] == \
        [(0, False), (1, False), (0, True), (1, False), (2, False)]
    assert [e.add_input for e in _spec(tiny.V_C).schedule] == [False] * 3      # no span
    assert [e.layer for e in _spec(tiny.V_D).schedule] == [0, 1, 2]             # run once
    assert plain.layer_order(tiny.V_A) == [(e.layer, e.add_input) for e in _spec(tiny.V_A).schedule]


def test_parts_and_their_constants():
    spec = _spec(tiny.V_A)
    ret, att = spec.layers[0].branches[0], spec.layers[1].branches[0]
    assert ret.part.kind == "retention" and ret.scale == 0.5 and ret.norm.kind == "rmsnorm"
    assert ret.part.params["decay"] == [0.9, 0.95, 0.99, 0.999]
    assert ret.part.params["position"] == {"kind": "rotary", "theta": 10000.0, "rotary_dim": 8,
                                           "pairing": "half"}
    p = att.part.params
    assert att.part.kind == "attention" and p["window"] == 9 and p["scale"] == 0.3
    assert p["sink"] == "mix.sink" and p["head_gate"] == "mix.g" and p["value_dim"] == 16
    assert spec.layers[1].branches[1].part.kind == "dense_mlp"
    assert spec.layers[1].branches[1].part.params["activation"] == "relu2"
    assert len(spec.layers[2].branches) == 1                      # no feed-forward
    assert spec.head.params["softcap"] == 8.0 and spec.head.params["tied"]
    assert spec.embedding.params["positions"] == {"name": "pos", "rows": 512}
    assert "softcap" not in _spec(tiny.V_C).head.params
    assert _spec(tiny.V_D).layers[2].branches[0].part.params["window"] == 0    # no mask


def test_manifest_names_and_shapes():
    names, ignorable = manifest(_spec(tiny.V_B))
    shapes = {k: v.shape for k, v in names.items()}
    assert shapes["embed"] == (130, 96) and shapes["pos"] == (512, 96)
    assert shapes["final.norm"] == (96,) and "head" in ignorable
    # attention: 6 heads on 2, keys of 16, values of 24
    for name, shape in {"l2.mix.q": (96, 96), "l2.mix.q.b": (96,), "l2.mix.k": (32, 96),
                        "l2.mix.k.b": (32,), "l2.mix.v": (48, 96), "l2.mix.v.b": (48,),
                        "l2.mix.q.norm": (16,), "l2.mix.k.norm": (16,), "l2.mix.sink": (6,),
                        "l2.mix.g": (6, 96), "l2.mix.o": (96, 144), "l2.norm1": (96,),
                        "l2.norm2": (96,), "l2.mlp.up": (64, 96), "l2.mlp.down": (96, 64),
                        # retention: 3 heads, keys of 16, values of 40
                        "l1.mix.q": (48, 96), "l1.mix.k": (48, 96), "l1.mix.v": (120, 96),
                        "l1.mix.g": (120, 96), "l1.mix.o": (96, 120)}.items():
        assert shapes[name] == shape, name
    assert not any(k.startswith("l1.mix.q.") or k.endswith("mlp.gate") for k in shapes)
    names, _ = manifest(_spec(tiny.V_A))
    assert "l2.norm2" not in names and "l2.mlp.up" not in names


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.9]), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.9, 0.9, 0.9, 1.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=3), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_refusals(edit, what):
    cfg = copy.deepcopy(tiny.V_A)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        virorax_config_from_dict(cfg)
    assert what in str(e.value)


def test_cache_requests_of_every_run():
    """Every run of a repeated layer asks for a cache or a state of its own."""
    from cretif_b200.cache import KVRequest, StateRequest
    from cretif_b200.engine.model import Model
    model = Model(_spec(tiny.V_A), torch.float32, "cpu")
    reqs = model.cache_requests()
    kinds = [type(reqs[(i, 0)]).__name__ for i in range(8)]
    assert kinds == ["StateRequest", "KVRequest", "StateRequest", "KVRequest", "StateRequest",
                     "KVRequest", "StateRequest", "KVRequest"]
    assert reqs[(1, 0)] == reqs[(3, 0)] == KVRequest(2, 16, 9)
    assert reqs[(0, 0)] == StateRequest((4 * 16 * 24,), torch.float32)
    assert reqs[(7, 0)] == KVRequest(4, 16, 21)
    # values of another size than the keys
    reqs = Model(_spec(tiny.V_B), torch.float32, "cpu").cache_requests()
    assert reqs[(4, 0)] == KVRequest(2, 16, 130, value_dim=24)


# ------------------------------------------------------------------ the plain implementation
def test_retention_forgets_by_its_decay():
    """One write, then empty keys: the read-out of the first value fades by g per step."""
    S, d, e = 6, 4, 3
    q = torch.zeros(S, 2, d, dtype=torch.float64)
    k = torch.zeros(S, 2, d, dtype=torch.float64)
    v = torch.zeros(S, 2, e, dtype=torch.float64)
    k[0, :, 1] = 1.0
    v[0] = torch.tensor([1.0, 2.0, 3.0])
    q[:, :, 1] = 1.0
    o = plain.retention(q, k, v, torch.tensor([0.5, 1.0], dtype=torch.float64))
    for t in range(S):
        assert torch.allclose(o[t, 0], v[0, 0] * 0.5 ** t)
        assert torch.allclose(o[t, 1], v[0, 1])              # a decay of one keeps everything


def test_retention_is_decayed_linear_attention():
    g = torch.Generator().manual_seed(1)
    S, H, d, e = 9, 2, 5, 4
    q, k = (torch.randn(S, H, d, generator=g, dtype=torch.float64) for _ in range(2))
    v = torch.randn(S, H, e, generator=g, dtype=torch.float64)
    decay = torch.tensor([0.8, 0.95], dtype=torch.float64)
    o = plain.retention(q, k, v, decay)
    for h in range(H):
        for t in range(S):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want)


def test_rotation_of_the_front_channels():
    g = torch.Generator().manual_seed(2)
    z = torch.randn(7, 3, 10, generator=g, dtype=torch.float64)
    r = plain.rotate_front(z, 100.0, 6)
    assert torch.equal(r[..., 6:], z[..., 6:])                   # the rest passes
    assert torch.equal(r[0], z[0])                               # position 0: angle 0
    assert torch.allclose((r[..., :6] ** 2).sum(-1), (z[..., :6] ** 2).sum(-1))
    # channel i is paired with channel i + 3; pair 0 turns by p, pair 1 by p * 100^(-1/3)
    p, i = 4, 1
    a = p * 100.0 ** (-2.0 * i / 6)
    u, w = z[p, 0, i], z[p, 0, i + 3]
    assert math.isclose(r[p, 0, i], u * math.cos(a) - w * math.sin(a), rel_tol=1e-12)
    assert math.isclose(r[p, 0, i + 3], w * math.cos(a) + u * math.sin(a), rel_tol=1e-12)
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 6, generator=g, dtype=torch.float64), \
        torch.randn(1, 1, 6, generator=g, dtype=torch.float64)
    s1 = plain.rotate_front(q, 50.0, 6, first_pos=9)[0, 0] @ plain.rotate_front(k, 50.0, 6, first_pos=4)[0, 0]
    s2 = plain.rotate_front(q, 50.0, 6, first_pos=25)[0, 0] @ plain.rotate_front(k, 50.0, 6, first_pos=20)[0, 0]
    assert math.isclose(float(s1), float(s2), rel_tol=1e-9)


def test_sink_takes_weight_but_gives_nothing():
    s = torch.tensor([[0.0, -math.inf], [1.0, 2.0]], dtype=torch.float64)
    vis = torch.tensor([[True, False], [True, True]])
    w = plain.softmax_with_sink(s, vis, torch.tensor(0.0, dtype=torch.float64))
    assert torch.allclose(w[0], torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert math.isclose(float(w[1].sum()), (math.e + math.e ** 2) / (1 + math.e + math.e ** 2))
    w = plain.softmax_with_sink(s, vis, torch.tensor(-50.0, dtype=torch.float64))
    assert torch.allclose(w.sum(-1), torch.ones(2, dtype=torch.float64))
    w = plain.softmax_with_sink(s, vis, torch.tensor(50.0, dtype=torch.float64))
    assert float(w.abs().max()) < 1e-20


def test_window_activation_and_cap():
    vis = plain.window_mask(5, 2)
    assert vis.tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                            [False, True, True, False, False], [False, False, True, True, False],
                            [False, False, False, True, True]]
    z = torch.tensor([-2.0, 0.0, 0.5, 3.0], dtype=torch.float64)
    assert plain.relu_squared(z).tolist() == [0.0, 0.0, 0.25, 9.0]
    c = plain.soft_cap(torch.tensor([-1e3, 0.1, 1e3], dtype=torch.float64), 5.0)
    assert abs(float(c[0]) + 5.0) < 1e-9 and abs(float(c[2]) - 5.0) < 1e-9
    assert abs(float(c[1]) - 0.1) < 1e-4


def test_a_further_pass_gets_the_input_again():
    """The plain model with a span run twice equals the layers spelled out by hand."""
    from cretif_b200.weights.loader import random_weights
    cfg = tiny.one_layer("retention", loop=(0, 1, 2), mult=0.7)
    names, _ = manifest(_spec(cfg))
    W = {k: v.double() for k, v in random_weights(names, 5, torch.bfloat16).items()}
    ids = [3, 9, 1, 40]
    streams = []
    plain.forward(cfg, W, ids, streams=streams)
    x0 = torch.stack([W["embed"][t] + W["pos"][p] for p, t in enumerate(ids)])
    m = cfg["layers"][0]["mixer"]

    def layer(x):
        return x + 0.7 * plain.mixer_retention(plain.unit(x, 1e-5) * W["l0.norm1"], W, "l0.mix.",
                                               m, 1e-5)
    x1 = layer(x0)
    assert torch.allclose(streams[0], x1)
    assert torch.allclose(streams[1], layer(x1 + x0))


def test_the_bench_configurations_build():
    """The models `bench.py --design virorax` measures parse and give a schedule with as many
    layer runs as the models beside them have layers."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    mod_spec = importlib.util.spec_from_file_location("bench_for_test", path)
    bench = importlib.util.module_from_spec(mod_spec)
    mod_spec.loader.exec_module(bench)
    for size, z in bench.DESIGN_SIZES.items():
        for layers in (4, 8):
            for name, cfg in bench.virorax_configs(z, layers).items():
                if not name.startswith("virorax"):
                    continue
                spec = _spec(cfg)
                spec.validate()
                assert len(spec.schedule) == layers, (size, name)
                assert spec.architecture == "Virorax"
