"""Typed configuration of the Virorax decoder, read from config.json, and its ModelSpec.

A Virorax checkpoint's config.json names its class with ``"architecture": "Virorax"`` and
describes the model as a list of layers, each with a mixer of its own kind and sizes:

=====================  ========================================================================
key                    meaning
=====================  ========================================================================
vocab, width           vocabulary and residual width
max_positions          rows of the learned position table (the longest sequence)
norm.eps               eps of every RMS norm of the model
residual_mult          factor on what every sublayer adds to the residual stream
logit_softcap          c: logits leave as c * tanh(logits / c)
loop                   ``{"start", "stop", "times"}``: layers start .. stop-1 run ``times`` times
                       in a row with the same tensors, each pass on caches and states of its own
layers[i].type         ``attention`` | ``retention``
layers[i].mixer        attention: heads, kv_heads, dim, vdim, scale, mask.size (window),
                       rot.base, rot.dims;  retention: heads, dim, vdim, decay (a number per
                       head), rot.base, rot.dims
layers[i].mlp          ``{"kind": "dense", "ff": F}`` or null for a layer without feed-forward
=====================  ========================================================================

The block is pre-norm: ``x += m * mixer(norm1(x))``, then ``x += m * ff(norm2(x))`` with
``m = residual_mult``; the input of layer 0 is the token's embedding row plus a learned vector
for its position, and before every pass of the repeated span but the first that input is added
to the stream again.  Tensors are named ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.norm1/2``,
``embed`` (also the output matrix), ``pos`` and ``final.norm``.  The two mixers map to the parts
``attention`` (with biases, a norm per head, a rotation of part of each head, a learned sink and
a per-head output gate) and ``retention``; the feed-forward is ``dense_mlp`` with the squared
relu.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .spec import BranchSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("attention", "retention")
FF_ACTIVATION = "relu2"                 # the design's dense feed-forward squares a relu


@dataclass
class ViroraxConfig:
    vocab: int
    width: int
    eps: float
    max_positions: int
    layers: List[Dict[str, Any]] = field(default_factory=list)
    residual_mult: float = 1.0
    logit_softcap: Optional[float] = None
    loop: Optional[Dict[str, int]] = None
    architecture: str = "Virorax"

    def layer_runs(self) -> List[tuple]:
        """(layer, starts a further pass) for every layer run, in order."""
        n = len(self.layers)
        loop = self.loop or {"start": 0, "stop": 0, "times": 1}
        a, b, times = loop["start"], loop["stop"], loop["times"]
        runs = [(i, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t > 0 and i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                             "width": self.width, "max_positions": self.max_positions,
                             "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
                             "layers": [dict(l) for l in self.layers]}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        return d


def _positive_int(where: str, d: Any, key: str) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}: {key} must be a positive integer, got {v!r}")
    return v


def _number(where: str, d: Any, key: str, positive: bool = False) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{where}: {key} must be a {'positive ' if positive else ''}number, "
                          f"got {v!r}")
    return float(v)


def _check_rot(where: str, m: Dict[str, Any]) -> None:
    rot = m.get("rot")
    if rot is None:
        return
    dims = _positive_int(where + ".rot", rot, "dims")
    _number(where + ".rot", rot, "base", positive=True)
    if dims % 2 or dims > m["dim"]:
        raise ConfigError(f"{where}.rot: dims ({dims}) must be even and at most dim ({m['dim']})")


def _check_mixer(i: int, kind: str, m: Any) -> None:
    where = f"layers[{i}].mixer"
    if not isinstance(m, dict):
        raise ConfigError(f"{where} must be an object")
    heads = _positive_int(where, m, "heads")
    _positive_int(where, m, "dim")
    _positive_int(where, m, "vdim")
    _check_rot(where, m)
    if kind == "attention":
        g = _positive_int(where, m, "kv_heads")
        if heads % g:
            raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({g})")
        _number(where, m, "scale", positive=True)
        if m.get("mask") is not None:               # no mask: every earlier key is seen
            _positive_int(where + ".mask", m["mask"], "size")
    else:
        decay = m.get("decay")
        if (not isinstance(decay, list) or len(decay) != heads
                or any(isinstance(g, bool) or not isinstance(g, (int, float)) or not 0 < g <= 1
                       for g in decay)):
            raise ConfigError(f"{where}: decay must list a number in (0, 1] for each of the "
                              f"{heads} heads, got {decay!r}")


def virorax_config_from_dict(raw: Dict[str, Any]) -> ViroraxConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm", "max_positions") if k not in raw]
    if missing:
        raise ConfigError(f"config.json lacks required keys: {missing}")
    vocab = _positive_int("config", raw, "vocab")
    width = _positive_int("config", raw, "width")
    max_positions = _positive_int("config", raw, "max_positions")
    eps = _number("norm", raw["norm"], "eps", positive=True)
    layers = raw["layers"]
    if not isinstance(layers, list) or not layers:
        raise ConfigError("layers must be a non-empty list")
    for i, layer in enumerate(layers):
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"layers[{i}].type must be one of {MIXER_TYPES}, got "
                              f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
        _check_mixer(i, layer["type"], layer.get("mixer"))
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"layers[{i}].mlp.kind must be 'dense', got {mlp!r}")
            _positive_int(f"layers[{i}].mlp", mlp, "ff")
    mult = 1.0 if raw.get("residual_mult") is None else _number("config", raw, "residual_mult")
    cap = None if raw.get("logit_softcap") is None else _number("config", raw, "logit_softcap",
                                                                positive=True)
    loop = raw.get("loop")
    if loop is not None:
        start = loop.get("start") if isinstance(loop, dict) else None
        if isinstance(start, bool) or not isinstance(start, int) or start < 0:
            raise ConfigError(f"loop.start must be a layer index, got {loop!r}")
        stop = _positive_int("loop", loop, "stop")
        times = _positive_int("loop", loop, "times")
        if not start < stop <= len(layers):
            raise ConfigError(f"loop: layers {start} .. {stop - 1} are not among the "
                              f"{len(layers)} layers")
        loop = {"start": start, "stop": stop, "times": times}
    return ViroraxConfig(vocab=vocab, width=width, eps=eps, max_positions=max_positions,
                         layers=[dict(l) for l in layers], residual_mult=mult, logit_softcap=cap,
                         loop=loop, architecture=str(raw.get("architecture", "Virorax")))


def _position(m: Dict[str, Any]) -> Dict[str, Any]:
    rot = m.get("rot")
    if rot is None:
        return {"kind": "none"}
    return {"kind": "rotary", "theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
            "pairing": "half"}


def _mixer_spec(kind: str, m: Dict[str, Any], eps: float) -> PartSpec:
    if kind == "attention":
        return PartSpec("attention", {
            "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "scale": float(m["scale"]),
            "window": (m.get("mask") or {}).get("size", 0), "position": _position(m),
            "bias": {"q": "mix.q.b", "k": "mix.k.b", "v": "mix.v.b"},
            "head_norm": {"eps": eps, "q": "mix.q.norm", "k": "mix.k.norm"},
            "sink": "mix.sink", "head_gate": "mix.g",
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o"}})
    return PartSpec("retention", {
        "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "decay": [float(g) for g in m["decay"]], "eps": eps, "position": _position(m),
        "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "o": "mix.o"}})


def build_virorax_spec(cfg: ViroraxConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"eps": cfg.eps, "name": name})

    layers: List[LayerSpec] = []
    for i, layer in enumerate(cfg.layers):
        branches = [BranchSpec("mixer", _mixer_spec(layer["type"], layer["mixer"], cfg.eps),
                               norm=norm("norm1"), scale=cfg.residual_mult)]
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = PartSpec("dense_mlp", {"intermediate_size": mlp["ff"],
                                        "activation": FF_ACTIVATION,
                                        "names": {"up": "mlp.up", "down": "mlp.down"}})
            branches.append(BranchSpec("feed_forward", ff, norm=norm("norm2"),
                                       scale=cfg.residual_mult))
        layers.append(LayerSpec(f"l{i}.", tuple(branches)))
    # every run of a layer is a schedule entry with caches and states of its own
    schedule = [ScheduleEntry(i, add_input=again) for i, again in cfg.layer_runs()]
    head = {"tied": True, "name": "head", "tied_to": "embed"}
    if cfg.logit_softcap is not None:
        head["softcap"] = cfg.logit_softcap
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding",
                           {"name": "embed",
                            "positions": {"name": "pos", "rows": cfg.max_positions}}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", head), max_positions=cfg.max_positions)


register_architecture("Virorax", virorax_config_from_dict, build_virorax_spec)
