"""Mipurax without a GPU: configuration, spec and manifest, refusals, and the plain
implementation's own properties."""
import copy
import math

import pytest
import torch

import mipurax_tiny as tiny
import plain_mipurax as plain
from cretif_b200.config import (ConfigError, build_mipurax_spec, mipurax_config_from_dict,
                                resolve_architecture)
from cretif_b200.engine.model import manifest


def _spec(cfg):
    return build_mipurax_spec(mipurax_config_from_dict(cfg))


def test_registered_and_parsed():
    assert resolve_architecture("Mipurax").config_from_dict is mipurax_config_from_dict
    cfg = mipurax_config_from_dict(tiny.M_A)
    assert (cfg.vocab, cfg.width, cfg.eps, len(cfg.layers)) == (96, 64, 1e-5, 4)
    assert mipurax_config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_parts_and_their_constants():
    spec = _spec(tiny.M_A)
    spec.validate()
    lat, att, lat2, reader = (spec.layers[i].branches[0] for i in range(4))
    assert all(b.norm.kind == "rmsnorm" and b.norm.params["offset"] == 1.0 and b.post_norm is None
               for layer in spec.layers for b in layer.branches)
    p = lat.part.params
    assert lat.part.kind == "latent_attention" and p["gate"] == "channel"
    assert (p["q_rank"], p["latent_rank"], p["rot_dim"], p["head_dim"], p["value_dim"]) == \
        (40, 24, 8, 16, 24)
    assert p["position"] == {"kind": "rotary", "theta": 10000.0, "rotary_dim": 8,
                             "pairing": "interleaved"}
    assert "sink" not in p["names"] and p["window"] == 0
    p2 = lat2.part.params
    assert p2["gate"] == "head" and p2["names"]["sink"] == "mix.sink"
    assert p2["position"]["pairing"] == "half" and p2["position"]["theta"] == 500.0
    pa = att.part.params
    assert att.part.kind == "attention" and pa["chunk"] == 9 and pa["window"] == 0
    assert pa["distance_slope"] == {"exponent": 8.0} and pa["own_kv"] and pa["scale"] == 0.3
    assert pa["position"] == {"kind": "none"}
    assert not reader.part.params["own_kv"] and reader.part.params["chunk"] == 21
    assert [e.cache for e in spec.schedule] == [None, None, None, 1]
    moe = spec.layers[1].branches[1].part
    assert moe.kind == "routed_experts" and not moe.params["gated"]
    assert moe.params["activation"] == "gelu" and moe.params["weight_on"] == "output"
    assert moe.params["renormalize"] and moe.params["sum_eps"] == 1e-20
    assert moe.params["groups"] == {"count": 4, "keep": 2}
    assert moe.params["shared"]["intermediate_size"] == 48
    dense = spec.layers[0].branches[1].part
    assert dense.kind == "dense_mlp" and dense.params["activation"] == "gelu"
    assert len(spec.layers[2].branches) == 1                          # no feed-forward
    assert spec.head.params["tied"]
    assert spec.embedding.params["norm"] == {"name": "embed.norm", "eps": 1e-5, "offset": 1.0}
    plain_moe = _spec(tiny.M_B).layers[0].branches[1].part.params
    assert "groups" not in plain_moe and "shared" not in plain_moe


def test_manifest_names_and_shapes():
    names, ignorable = manifest(_spec(tiny.M_A))
    shapes = {k: v.shape for k, v in names.items()}
    for name, shape in {
            "embed": (96, 64), "embed.norm": (64,), "final.norm": (64,),
            # the queries' latent 40, two heads of 16 flat + 8 rotated, latent 24, values of 24
            "l0.mix.dq": (40, 64), "l0.mix.dq.norm": (40,), "l0.mix.uq": (48, 40),
            "l0.mix.dkv": (32, 64), "l0.mix.dkv.norm": (24,), "l0.mix.uk": (32, 24),
            "l0.mix.uv": (48, 24), "l0.mix.g": (48, 64), "l0.mix.o": (64, 48),
            "l0.mlp.up": (96, 64), "l0.mlp.down": (64, 96),
            "l1.mix.q": (64, 64), "l1.mix.k": (32, 64), "l1.mix.v": (32, 64),
            "l1.mix.o": (64, 64), "l1.mlp.router": (8, 64), "l1.mlp.e7.up": (32, 64),
            "l1.mlp.e0.down": (64, 32), "l1.mlp.shared.up": (48, 64),
            "l1.mlp.shared.down": (64, 48),
            # four heads of 8 + 16, latent 48, a gate and a sink per head
            "l2.mix.uq": (96, 24), "l2.mix.dkv": (64, 64), "l2.mix.g": (4, 64),
            "l2.mix.sink": (4,), "l2.mix.o": (64, 32),
            "l3.mix.q": (64, 64), "l3.mix.o": (64, 64)}.items():
        assert shapes[name] == shape, name
    assert "head" in ignorable
    for absent in ("l3.mix.k", "l3.mix.v", "l0.mix.sink", "l2.norm2", "l2.mlp.up",
                   "l1.mlp.e0.gate", "l1.mlp.e8.up", "l0.mix.q"):
        assert absent not in shapes, absent


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="retention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("mask"), "size"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=8), "differs"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=5), "groups"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_refusals(edit, text):
    cfg = copy.deepcopy(tiny.M_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        mipurax_config_from_dict(cfg)


def test_a_reader_of_a_reader_is_refused():
    cfg = copy.deepcopy(tiny.M_D)
    cfg["layers"][3]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="no keys and values"):
        mipurax_config_from_dict(cfg)


# ------------------------------------------------------------------ the plain implementation
def test_masks_and_slopes():
    m = plain.chunk_mask(10, 4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert m[4].tolist() == [False] * 4 + [True] + [False] * 5      # a chunk's first position
    assert m[3].tolist() == [True] * 4 + [False] * 6
    assert plain.chunk_mask(7, 1).sum() == 7 and torch.equal(plain.chunk_mask(6, 50),
                                                             plain.causal_mask(6))
    s = plain.distance_slopes(4)
    assert torch.allclose(s, torch.tensor([0.25, 0.0625, 2.0 ** -6, 2.0 ** -8], dtype=s.dtype))
    assert float(plain.distance_slopes(1)[0]) == 2.0 ** -8


def test_softmax_with_a_sink():
    scores = torch.tensor([[[0.0, 1.0], [2.0, -1.0]]], dtype=torch.float64)
    vis = plain.causal_mask(2)
    p = plain.softmax_rows(scores, vis)
    assert torch.allclose(p.sum(-1), torch.ones(1, 2, dtype=torch.float64))
    q = plain.softmax_rows(scores, vis, sink=torch.tensor([0.0], dtype=torch.float64))
    assert abs(float(q[0, 0, 0]) - 0.5) < 1e-12                      # e^0 / (e^0 + e^0)
    e2, em1 = math.exp(2.0), math.exp(-1.0)
    assert abs(float(q[0, 1].sum()) - (e2 + em1) / (e2 + em1 + 1.0)) < 1e-12
    far = plain.softmax_rows(scores, vis, sink=torch.tensor([-50.0], dtype=torch.float64))
    assert torch.allclose(far, p)
    loud = plain.softmax_rows(scores, vis, sink=torch.tensor([50.0], dtype=torch.float64))
    assert float(loud.sum()) < 1e-15


def test_rotation_layouts():
    g = torch.Generator().manual_seed(0)
    z = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    for layout in ("interleaved", "half"):
        r = plain.rotate(z, 100.0, 8, layout)
        assert torch.equal(r[..., 8:], z[..., 8:]) and torch.equal(r[0], z[0])    # position 0
        assert torch.allclose((r ** 2).sum(-1), (z ** 2).sum(-1))
        shifted = plain.rotate(z[1:], 100.0, 8, layout, first_pos=1)
        assert torch.allclose(shifted, r[1:])
    # pair 1 turns by p * base^(-2/8): channels (2, 3) interleaved, (1, 5) in halves
    a = 3 * 100.0 ** (-0.25)
    u, v = z[3, 0, 2], z[3, 0, 3]
    r = plain.rotate(z, 100.0, 8, "interleaved")
    assert abs(float(r[3, 0, 2]) - float(u * math.cos(a) - v * math.sin(a))) < 1e-12
    assert abs(float(r[3, 0, 3]) - float(v * math.cos(a) + u * math.sin(a))) < 1e-12
    u, v = z[3, 0, 1], z[3, 0, 5]
    r = plain.rotate(z, 100.0, 8, "half")
    assert abs(float(r[3, 0, 1]) - float(u * math.cos(a) - v * math.sin(a))) < 1e-12
    assert abs(float(r[3, 0, 5]) - float(v * math.cos(a) + u * math.sin(a))) < 1e-12


def test_routing_by_groups():
    # six experts in three groups of two; scores chosen through their logits
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.8, 0.05]], dtype=torch.float64)
    x = torch.log(s / (1 - s))                       # a router that is the identity
    router = torch.eye(6, dtype=torch.float64)
    rule = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    chosen, w = plain.route(x, router, rule)         # group sums 1.0, 1.15, 0.85
    assert sorted(chosen[0].tolist()) == [2, 3]
    assert abs(float(w.sum()) - 1.0) < 1e-12 and abs(float(w[0].max()) - 0.6 / 1.15) < 1e-12
    rule["groups"]["keep"] = 2                       # groups 1 and 0: the best two of 0..3
    chosen, w = plain.route(x, router, rule)
    assert sorted(chosen[0].tolist()) == [0, 2]
    assert abs(float(w[0].max()) - 0.9 / 1.5) < 1e-12
    chosen, _ = plain.route(x, router, {"experts": 6, "top": 2})        # no groups
    assert sorted(chosen[0].tolist()) == [0, 4]


def test_a_reader_uses_its_writers_keys_and_values():
    """The last layer of A computes with layer 1's keys and values: given the writer's input
    it equals a layer with copies of the writer's projections, given another input it does not."""
    from cretif_b200.weights.loader import random_weights
    names, _ = manifest(_spec(tiny.M_A))
    w = {k: v.double() for k, v in random_weights(names, 3, torch.bfloat16).items()}
    x = torch.randn(30, 64, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    m1, m3 = tiny.M_A["layers"][1]["mixer"], tiny.M_A["layers"][3]["mixer"]
    _, kv = plain.chunked_attention(x, w, "l1.mix.", m1)
    x3 = torch.randn(30, 64, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    got, _ = plain.chunked_attention(x3, w, "l3.mix.", m3, kv=kv)
    w2 = dict(w)
    w2["l3.mix.k"], w2["l3.mix.v"] = w["l1.mix.k"], w["l1.mix.v"]
    own, _ = plain.chunked_attention(x, w2, "l3.mix.", dict(m3, kv_from=None))
    # with the writer's input as its own input the reader's keys and values are the same
    again, _ = plain.chunked_attention(x, w, "l3.mix.", m3, kv=kv)
    assert torch.allclose(own, again)
    assert not torch.allclose(got, again)


def test_cache_requests_of_a_reader():
    from cretif_b200.engine.model import Model
    model = Model(_spec(tiny.M_A), torch.float32, "cpu")       # built, not loaded
    reqs = model.cache_requests()
    assert (3, 0) not in reqs and (1, 0) in reqs                     # the reader asks for none
    assert reqs[(0, 0)].head_dim == 32 and reqs[(0, 0)].shared_values
    assert reqs[(2, 0)].head_dim == 64 and reqs[(1, 0)].num_kv_heads == 2
