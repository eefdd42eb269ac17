"""Typed configuration of the Mipurax decoder, read from config.json, and its ModelSpec.

A Mipurax checkpoint's config.json names its class with ``"architecture": "Mipurax"`` and
describes the model as a list of layers, each with a mixer of its own kind and sizes:

=====================  ========================================================================
key                    meaning
=====================  ========================================================================
vocab, width           vocabulary and residual width
norm.eps               eps of every RMS norm of the model
layers[i].type         ``latent_attention`` | ``latent_attention_2`` | ``attention``
layers[i].mixer        latent kinds: heads, dim (flat query/key size per head), rot_dim (size of
                       the rotated part), vdim, kv_rank, q_rank, scale, rot {base, dims} (dims:
                       how many of the part's first channels turn; the design has all);
                       attention: heads, kv_heads, dim, vdim, scale, mask.size (the chunk),
                       kv_from (optional: the layer whose keys and values this layer reads
                       instead of projecting its own)
layers[i].mlp          ``{"kind": "dense", "ff": F}``, ``{"kind": "moe", "expert": {"ff": F},
                       "router": {"experts": E, "top": k, "groups": {"count", "keep"}},
                       "shared": {"ff": Fs}}`` (groups and shared optional), or null
max_positions          (optional) longest sequence; the design itself has no limit
=====================  ========================================================================

The embedding's rows pass an RMS norm (``embed.norm``) before the first layer.  A block is
pre-norm: ``x += mixer(norm1(x))``, ``x += ff(norm2(x))``; the block's norms, the embedding's and
the final one store their weights around zero (factor ``1 + w``), the norms inside the mixers
store the factor itself.  The output matrix is the embedding table.  Tensors are named
``l<i>.mix.*``, ``l<i>.mlp.*`` (``e<n>.up/down``, ``router``, ``shared.up/down``),
``l<i>.norm1/2``, ``embed``, ``embed.norm`` and ``final.norm``.

The two latent kinds differ in what the design fixes for them: ``latent_attention`` rotates
neighbouring channels (2i, 2i + 1), has an ordinary softmax and gates its output channel by
channel; ``latent_attention_2`` rotates channels i and i + dims/2, has a learned term per head in
the softmax's denominator and gates head by head.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List

from .registry import ConfigError, register_architecture
from .spec import BranchSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("latent_attention", "latent_attention_2", "attention")
DEFAULT_MAX_POSITIONS = 1 << 20
# what the design fixes
SLOPE_EXPONENT = 8.0                     # head h takes 2^(-8 (h + 1) / heads) per position off
FF_ACTIVATION = "gelu"                   # the exact form, dense layers and experts alike
WEIGHT_SUM_EPS = 1e-20                   # added to the sum of a token's chosen scores
LATENT_KINDS = {
    "latent_attention": {"pairing": "interleaved", "sink": False, "gate": "channel"},
    "latent_attention_2": {"pairing": "half", "sink": True, "gate": "head"},
}


@dataclass
class MipuraxConfig:
    vocab: int
    width: int
    eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Mipurax"

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                             "width": self.width, "norm": {"eps": self.eps},
                             "layers": [dict(l) for l in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
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


def _check_latent(i: int, m: Dict[str, Any]) -> None:
    where = f"layers[{i}].mixer"
    for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
        _positive_int(where, m, key)
    _number(where, m, "scale", positive=True)
    rot = m.get("rot")
    _number(where + ".rot", rot, "base", positive=True)
    dims = _positive_int(where + ".rot", rot, "dims")
    if dims > m["rot_dim"] or dims % 2:
        raise ConfigError(f"{where}: rot.dims ({dims}) must be even and at most rot_dim "
                          f"({m['rot_dim']}): the rotation turns the first channels of the "
                          "rotated part")


def _check_attention(i: int, m: Dict[str, Any], layers: List[Any]) -> None:
    where = f"layers[{i}].mixer"
    heads = _positive_int(where, m, "heads")
    g = _positive_int(where, m, "kv_heads")
    if heads % g:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({g})")
    _positive_int(where, m, "dim")
    _positive_int(where, m, "vdim")
    _number(where, m, "scale", positive=True)
    _positive_int(where + ".mask", m.get("mask"), "size")
    j = m.get("kv_from")
    if j is not None:
        if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
            raise ConfigError(f"{where}: kv_from must name an earlier layer, got {j!r}")
        other = layers[j]
        om = other.get("mixer") if isinstance(other, dict) else None
        if (not isinstance(other, dict) or other.get("type") != "attention"
                or not isinstance(om, dict) or om.get("kv_from") is not None):
            raise ConfigError(f"{where}: kv_from = {j}: that layer stores no keys and values of "
                              "its own")
        for key in ("kv_heads", "dim", "vdim"):
            if om.get(key) != m.get(key):
                raise ConfigError(f"{where}: kv_from = {j}: {key} differs ({om.get(key)!r} there, "
                                  f"{m.get(key)!r} here)")


def _check_mlp(i: int, mlp: Any) -> None:
    where = f"layers[{i}].mlp"
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind", "dense") not in ("dense", "moe"):
        raise ConfigError(f"{where}.kind must be 'dense' or 'moe', got {mlp!r}")
    if mlp.get("kind", "dense") == "dense":
        _positive_int(where, mlp, "ff")
        return
    _positive_int(where + ".expert", mlp.get("expert"), "ff")
    router = mlp.get("router")
    n = _positive_int(where + ".router", router, "experts")
    top = _positive_int(where + ".router", router, "top")
    if top > n:
        raise ConfigError(f"{where}.router: top ({top}) exceeds experts ({n})")
    groups = router.get("groups")
    if groups is not None:
        count = _positive_int(where + ".router.groups", groups, "count")
        keep = _positive_int(where + ".router.groups", groups, "keep")
        if n % count or keep > count or keep * (n // count) < top:
            raise ConfigError(f"{where}.router.groups: {n} experts do not form {count} equal "
                              f"groups of which {keep} hold {top} experts")
    if mlp.get("shared") is not None:
        _positive_int(where + ".shared", mlp["shared"], "ff")


def mipurax_config_from_dict(raw: Dict[str, Any]) -> MipuraxConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
    if missing:
        raise ConfigError(f"config.json lacks required keys: {missing}")
    vocab = _positive_int("config", raw, "vocab")
    width = _positive_int("config", raw, "width")
    eps = _number("norm", raw["norm"], "eps", positive=True)
    layers = raw["layers"]
    if not isinstance(layers, list) or not layers:
        raise ConfigError("layers must be a non-empty list")
    for i, layer in enumerate(layers):
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"layers[{i}].type must be one of {MIXER_TYPES}, got "
                              f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
        m = layer.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"layers[{i}].mixer must be an object")
        if layer["type"] == "attention":
            _check_attention(i, m, layers)
        else:
            _check_latent(i, m)
        _check_mlp(i, layer.get("mlp"))
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"max_positions must be a positive integer, got {max_positions!r}")
    return MipuraxConfig(vocab=vocab, width=width, eps=eps, layers=[dict(l) for l in layers],
                         max_positions=max_positions,
                         architecture=str(raw.get("architecture", "Mipurax")))


def _mixer_spec(kind: str, m: Dict[str, Any], eps: float) -> PartSpec:
    if kind == "attention":
        return PartSpec("attention", {
            "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "scale": float(m["scale"]), "window": 0,
            "chunk": int(m["mask"]["size"]), "distance_slope": {"exponent": SLOPE_EXPONENT},
            "position": {"kind": "none"}, "own_kv": m.get("kv_from") is None,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o"}})
    fixed = LATENT_KINDS[kind]
    names = {"q_down": "mix.dq", "q_norm": "mix.dq.norm", "q_up": "mix.uq", "down": "mix.dkv",
             "down_norm": "mix.dkv.norm", "up_k": "mix.uk", "up_v": "mix.uv", "gate": "mix.g",
             "o": "mix.o"}
    if fixed["sink"]:
        names["sink"] = "mix.sink"
    return PartSpec("latent_attention", {
        "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "latent_rank": m["kv_rank"], "q_rank": m["q_rank"], "rot_dim": m["rot_dim"],
        "scale": float(m["scale"]), "window": 0, "eps": eps, "gate": fixed["gate"],
        "position": {"kind": "rotary", "theta": float(m["rot"]["base"]),
                     "rotary_dim": int(m["rot"]["dims"]), "pairing": fixed["pairing"]},
        "names": names})


def _mlp_spec(mlp: Dict[str, Any]) -> PartSpec:
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("dense_mlp", {"intermediate_size": mlp["ff"],
                                      "activation": FF_ACTIVATION,
                                      "names": {"up": "mlp.up", "down": "mlp.down"}})
    router = mlp["router"]
    params: Dict[str, Any] = {
        "num_experts": router["experts"], "top": router["top"],
        "intermediate_size": mlp["expert"]["ff"], "gated": False, "activation": FF_ACTIVATION,
        "weight_on": "output", "renormalize": True, "sum_eps": WEIGHT_SUM_EPS,
        "names": {"router": "mlp.router", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}}
    if router.get("groups") is not None:
        params["groups"] = {"count": int(router["groups"]["count"]),
                            "keep": int(router["groups"]["keep"])}
    if mlp.get("shared") is not None:
        params["shared"] = {"intermediate_size": int(mlp["shared"]["ff"]),
                            "names": {"up": "mlp.shared.up", "down": "mlp.shared.down"}}
    return PartSpec("routed_experts", params)


def build_mipurax_spec(cfg: MipuraxConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"eps": cfg.eps, "name": name, "offset": 1.0})

    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(cfg.layers):
        branches = [BranchSpec("mixer", _mixer_spec(layer["type"], layer["mixer"], cfg.eps),
                               norm=norm("norm1"))]
        if layer.get("mlp") is not None:
            branches.append(BranchSpec("feed_forward", _mlp_spec(layer["mlp"]),
                                       norm=norm("norm2")))
        layers.append(LayerSpec(f"l{i}.", tuple(branches)))
        schedule.append(ScheduleEntry(i, cache=layer["mixer"].get("kv_from")))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", {
            "name": "embed", "norm": {"name": "embed.norm", "eps": cfg.eps, "offset": 1.0}}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"tied": True, "name": "head", "tied_to": "embed"}),
        max_positions=cfg.max_positions)


register_architecture("Mipurax", mipurax_config_from_dict, build_mipurax_spec)
