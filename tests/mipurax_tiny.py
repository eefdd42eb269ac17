"""Tiny Mipurax configurations for the tests; they differ in every size, order and option."""
import numpy as np


def _lat(heads, dim, rot, vdim, kv_rank, q_rank, scale, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank,
            "q_rank": q_rank, "scale": scale, "rot": {"base": base, "dims": dims or rot}}


def _att(heads, kv, dim, vdim, chunk, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": chunk}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _ff(n):
    return {"kind": "dense", "ff": n}


def _moe(experts, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _model(vocab, width, eps, layers, positions=1024):
    return {"architecture": "Mipurax", "vocab": vocab, "width": width, "max_positions": positions,
            "norm": {"eps": eps}, "layers": layers}


# every kind of layer; chunks of 9 and 21 keys; the last layer reads layer 1's keys and values
# with a chunk of its own; eight experts in four groups of which two are kept, a shared expert
M_A = _model(96, 64, 1e-5, [
    {"type": "latent_attention", "mixer": _lat(2, 16, 8, 24, 24, 40, 0.2), "mlp": _ff(96)},
    {"type": "attention", "mixer": _att(4, 2, 16, 16, 9, 0.3),
     "mlp": _moe(8, 2, 32, groups=(4, 2), shared=48)},
    {"type": "latent_attention_2", "mixer": _lat(4, 8, 16, 8, 48, 24, 0.25, 500.0), "mlp": None},
    {"type": "attention", "mixer": _att(4, 2, 16, 16, 21, 0.25, kv_from=1), "mlp": _ff(80)},
])
# sizes the tensor-core kernels take in bfloat16 (latent plus rotated part 96 and 128, heads of
# 64), chunks that cross cache blocks (70, 130), values wider and narrower than keys, experts
# without groups and without a shared one, one expert a token
M_B = _model(130, 96, 1e-6, [
    {"type": "attention", "mixer": _att(2, 1, 64, 64, 130, 0.15), "mlp": _moe(3, 1, 64)},
    {"type": "latent_attention", "mixer": _lat(3, 16, 32, 40, 64, 32, 0.2, 30.0), "mlp": _ff(64)},
    {"type": "attention", "mixer": _att(6, 2, 32, 16, 70, 0.2), "mlp": _ff(128)},
    {"type": "latent_attention_2", "mixer": _lat(2, 32, 16, 24, 112, 64, 0.15), "mlp": None},
])
# everything that can be one is one: one head, a chunk that shows a query nothing but itself, a
# chunk of two, one expert, groups of one expert each, a rotated part of one pair, a rotated part
# of which only the first pair turns
M_C = _model(70, 48, 1e-5, [
    {"type": "attention", "mixer": _att(1, 1, 8, 8, 1, 1.0), "mlp": _moe(1, 1, 16)},
    {"type": "latent_attention_2", "mixer": _lat(1, 8, 2, 8, 8, 8, 0.5), "mlp": _ff(48)},
    {"type": "attention", "mixer": _att(1, 1, 16, 8, 2, 0.5),
     "mlp": _moe(4, 2, 24, groups=(4, 3), shared=8)},
    {"type": "latent_attention", "mixer": _lat(1, 4, 4, 4, 12, 16, 0.4, dims=2), "mlp": None},
])
# sizes that are multiples of nothing in particular: head sizes 12 and 20, a width of 36, an odd
# vocabulary, ranks of 20 and 27; a chunk longer than any test sequence; every group kept; a
# reader right after its writer and a second reader of the same layer
M_D = _model(77, 36, 1e-5, [
    {"type": "attention", "mixer": _att(3, 1, 12, 20, 500, 0.29),
     "mlp": _moe(6, 3, 20, groups=(2, 2))},
    {"type": "attention", "mixer": _att(3, 1, 12, 20, 33, 0.3, kv_from=0), "mlp": None},
    {"type": "latent_attention", "mixer": _lat(3, 12, 6, 10, 20, 27, 0.3, 77.0), "mlp": _ff(56)},
    {"type": "attention", "mixer": _att(3, 1, 12, 20, 64, 0.2, kv_from=0), "mlp": _ff(24)},
])

CONFIGS = {"A": M_A, "B": M_B, "C": M_C, "D": M_D}
SEEDS = {"A": 11, "B": 12, "C": 13, "D": 14}


def tokens(name, n, seed):
    rng = np.random.default_rng(1000 * seed + n)
    return rng.integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def one_layer(kind, mixer=None, mlp=None, vocab=64, width=64):
    """A model of one layer of the given kind."""
    if mixer is None:
        mixer = _att(4, 2, 16, 16, 16, 0.25) if kind == "attention" \
            else _lat(4, 16, 8, 16, 32, 24, 0.2)
    return _model(vocab, width, 1e-5, [{"type": kind, "mixer": mixer, "mlp": mlp}],
                  positions=4096)
