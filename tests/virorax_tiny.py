"""Tiny Virorax configurations for the tests; they differ in every size, order and option."""
import numpy as np


def _att(heads, kv, dim, vdim, window, scale, rot_dims, base=10000.0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"base": base, "dims": rot_dims}}
    if window:
        m["mask"] = {"size": window}
    return m


def _ret(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
            "rot": {"base": base, "dims": rot_dims}}


def _ff(n):
    return {"kind": "dense", "ff": n}


def _model(vocab, width, eps, layers, mult=1.0, cap=None, loop=None, positions=512):
    cfg = {"architecture": "Virorax", "vocab": vocab, "width": width, "max_positions": positions,
           "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if cap is not None:
        cfg["logit_softcap"] = cap
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# retention first (value size unlike key size, part of a head rotated), a span of two layers run
# three times, an attention layer without feed-forward after it
V_A = _model(96, 64, 1e-5, [
    {"type": "retention", "mixer": _ret(4, 16, 24, [0.9, 0.95, 0.99, 0.999], 8), "mlp": _ff(96)},
    {"type": "attention", "mixer": _att(4, 2, 16, 16, 9, 0.3, 8), "mlp": _ff(80)},
    {"type": "retention", "mixer": _ret(2, 32, 16, [0.97, 0.6], 32, 500.0), "mlp": None},
    {"type": "attention", "mixer": _att(4, 4, 16, 16, 21, 0.25, 16), "mlp": None},
], mult=0.5, cap=8.0, loop=(1, 3, 3))
# windows that cross cache blocks (70, 130), values wider and narrower than keys, the repeated
# span starts at layer 0 and is the whole model but its last layer
V_B = _model(130, 96, 1e-6, [
    {"type": "attention", "mixer": _att(2, 1, 32, 32, 70, 0.2, 16), "mlp": _ff(64)},
    {"type": "retention", "mixer": _ret(3, 16, 40, [0.999, 0.98, 0.9], 4), "mlp": _ff(128)},
    {"type": "attention", "mixer": _att(6, 2, 16, 24, 130, 0.3, 16, 30.0), "mlp": _ff(64)},
], mult=0.8, cap=30.0, loop=(0, 2, 2))
# everything that can be one is one: one head, a window that shows a query nothing but itself,
# a window of two, a decay of one (nothing is forgotten), no repeated span, factor one, no cap
V_C = _model(70, 48, 1e-5, [
    {"type": "retention", "mixer": _ret(1, 8, 8, [1.0], 8), "mlp": None},
    {"type": "attention", "mixer": _att(1, 1, 8, 8, 1, 1.0, 2), "mlp": _ff(48)},
    {"type": "attention", "mixer": _att(1, 1, 16, 8, 2, 0.5, 16), "mlp": None},
])
# sizes that are multiples of nothing in particular: head sizes 12 and 20, a width of 40, an odd
# vocabulary; a window longer than any test sequence and a layer that sees every key; a span run
# once over is no repetition
V_D = _model(77, 40, 1e-5, [
    {"type": "attention", "mixer": _att(3, 1, 12, 20, 500, 0.29, 4), "mlp": _ff(56)},
    {"type": "retention", "mixer": _ret(3, 12, 6, [0.5, 0.9, 0.99], 12), "mlp": None},
    {"type": "attention", "mixer": _att(2, 2, 20, 6, 0, 0.3, 10), "mlp": _ff(24)},
], mult=1.3, cap=5.0, loop=(1, 2, 1))
# head sizes the tensor-core attention kernels take (64 without and with a window, 128), a wide
# retention head; the repeated span is the last layer alone
V_E = _model(200, 128, 1e-6, [
    {"type": "attention", "mixer": _att(4, 2, 64, 64, 100, 0.11, 32), "mlp": _ff(192)},
    {"type": "retention", "mixer": _ret(2, 64, 128, [0.99, 0.9], 16), "mlp": None},
    {"type": "attention", "mixer": _att(4, 1, 64, 64, 0, 0.12, 64), "mlp": None},
    {"type": "attention", "mixer": _att(2, 1, 128, 128, 40, 0.09, 64), "mlp": _ff(128)},
], mult=0.6, cap=20.0, loop=(3, 4, 2))
CONFIGS = {"A": V_A, "B": V_B, "C": V_C, "D": V_D, "E": V_E}
SEEDS = {"A": 111, "B": 222, "C": 333, "D": 444, "E": 555}


def one_layer(kind: str, window: int = 12, mixer=None, **kw):
    """A model of a single layer of one mixer and no feed-forward: the mechanism alone."""
    if mixer is None:
        mixer = {"attention": _att(4, 2, 16, 16, window, 0.4, 8),
                 "retention": _ret(4, 16, 8, [0.9, 0.95, 0.99, 0.999], 16)}[kind]
    return _model(80, 64, 1e-5, [{"type": kind, "mixer": mixer, "mlp": None}], positions=1024,
                  **kw)


def tokens(name: str, length: int, seed: int):
    rng = np.random.default_rng(9000 * seed + length)
    return rng.integers(0, CONFIGS[name]["vocab"], size=length).tolist()
