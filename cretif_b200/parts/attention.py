"""The attention mixer: grouped-query causal attention over the block cache.

Order of work as in the reference's block (src/attention.cu:542-731): q, k, v
projections without bias (:567-576, here one product with the three matrices
stacked), position encoding of q and k (:589-597), cache write (:607-608), scores
scaled after the dot product, causal mask, softmax, weighted sum of values
(:683-714), output projection (:720-728).  Unlike the reference there is no separate
score tensor and no transposition of the cache: the attention kernels read the
cache's blocks directly, for whole prompts and for single tokens alike.

Two options change what is projected and normed: ``qk_norm`` applies an RMS norm with a
weight per channel over the WHOLE query projection and over the whole key projection (all
heads of a token as one vector) before the heads are split; ``values: "keys"`` drops the value
projection, the values being the keys as projected, before that norm.  ``sink`` names a tensor
with one number per query head whose exponential joins the softmax's denominator
(``fixed_sink`` gives every head the same constant instead: 0 adds one to the denominator).

A second family of options serves attention whose projections pass a short causal
convolution over time: ``conv`` (taps and the tensors' names; the last taps - 1 projected
rows of a sequence are kept per cache slot), ``head_norm`` (q and k of every head divided by
their root mean square, no weight), ``query_gain`` (the query times
``1 + coef * ln(floor((pos + 1) / every) + 1)``), ``distance_bias`` (a learned table
``[rows, heads]`` added to the scaled scores by distance: a row per distance below rows/2,
beyond that rows spaced by the logarithm up to ``far``), ``value_dim`` (values of another
size than the keys) and ``own_kv: False`` (no key and value tensors: the layer reads the keys
and values that another schedule entry stores, with queries, bias and everything else of its
own).  One kernel does convolution, head norm, gain and the cache write.

``chunk`` (an integer) replaces the sliding window by chunks: a query sees the earlier keys of
its own run of ``chunk`` positions, runs counted from position 0 of the sequence.
``distance_slope`` (``{"exponent": x}``) takes ``slope_h * (i - j)`` off the scaled score of key j
for query i, with ``slope_h = 2^(-x (h + 1) / heads)``.  Both belong to the family whose
projections are handled head by head, which also serves a layer without key and value tensors of
its own (``own_kv: False``).
"""
from __future__ import annotations

import torch

from ..cache import KVRequest, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, build_part, register_part
from .linear import linear

_force_plain = False
_fused_steps = True
# Steps of at most this many tokens take the fused projection kernels; beyond 32 tokens they
# run as row groups of one launch (measured on a B200: a 64-token step at SmolLM2-135M sizes
# takes half the time of the tensor-core products, whose 128-row tiles run on a few CTAs).
FUSED_MAX_TOKENS = 64


def fused_steps_enabled() -> bool:
    return _fused_steps


def enable_fused_steps(on: bool) -> None:
    """Switch the fused few-token kernels on or off (tests compare both ways)."""
    global _fused_steps
    _fused_steps = bool(on)


def force_plain_attention(on: bool) -> None:
    """Use the one-warp-per-query kernel for every step (the tests' yardstick)."""
    global _force_plain
    _force_plain = bool(on)


def distance_edges(rows: int, far: float):
    """The smallest distance of every row of a distance-bias table: row n for n < rows/2, then
    ``rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2))`` capped at the last
    row.  Computed once on the host in 64-bit; the kernels only search the edges."""
    import numpy as np
    half = rows // 2
    if rows < 2 or not far > half:
        raise ValueError(f"distance bias: {rows} rows need far > {half}, got {far}")
    n = np.arange(half, int(np.ceil(far)) + 2, dtype=np.float64)
    bucket = np.minimum(rows - 1, half + np.floor(np.log(n / half) / np.log(far / half)
                                                  * (rows - half))).astype(np.int64)
    edges = np.arange(rows, dtype=np.int64)
    for b in range(half, rows):
        edges[b] = half + int(np.argmax(bucket >= b))      # reached at far at the latest
    return edges.astype(np.int32)


# The tensor-core kernels take a bias by distance as a dense table of its first distances (up
# to this many, in shared memory) plus one number for everything farther.
FAST_BIAS_MAX_DISTANCES = 4096


def run_attention(q, o, ctx, kv, nh, nkv, hd, scale, window, dtype, sink=None, vd=0, bias=None,
                  bias_edges=None, bias_dense=None, slope=None, slope_log2e=None):
    """Causal (windowed) attention of the step's queries ``q`` [T, nh·hd] over the cache view
    ``kv`` into ``o``, with the kernel that fits the step: the decode kernels when every
    sequence brings one token, the prompt kernel otherwise, the plain kernel for float32 and
    for whatever the fast ones do not take (values of another size than the keys, a bias whose
    rows reach farther than the fast kernels' table).  ``bias`` [rows, heads] with
    ``bias_edges`` is the bias by distance as the plain kernel takes it, ``bias_dense`` =
    (near [heads, n_far], far [heads]), times log2 e, as the tensor-core kernels do.  ``window``
    below zero stands for chunks of ``-window`` positions.  ``slope`` [heads]: a multiple of the
    distance taken off the scores; the plain kernel takes it as it is, the fast kernels work in
    powers of two and take ``slope_log2e``, the same numbers times log2 e."""
    vd = vd or hd
    fast = (not _force_plain and dtype == torch.bfloat16 and (sink is None or hd <= 128)
            and vd == hd and not (bias is not None and slope is not None)
            and (bias is None or (bias_dense is not None and hd <= 128))
            and (slope is None or (slope_log2e is not None and hd <= 128)))
    near, far = bias_dense if (bias is not None and bias_dense is not None) else (None, None)
    tilt = slope_log2e if slope is not None else None
    if fast:
        if ctx.is_decode and ops.attn_decode_supported(hd, kv.block_tokens, min(nh // nkv, 8)) \
                and (nh // nkv <= 8 or nkv == 1):
            # the kernel takes up to eight query heads per key/value head; more heads on ONE
            # key/value head (a shared latent) go as groups of eight in one launch whose items
            # are (sequence, group) pairs, where the rows allow that view ...
            G = nh // 8
            if (nh // nkv > 8 and nh % 8 == 0 and hd <= 128 and q.stride(0) == nh * hd
                    and o.stride(0) == nh * hd and ops.attn_decode_supported(hd, kv.block_tokens, 8)):
                key = ("decode_head_groups", G)
                if key not in ctx.extras:       # once a step, for every layer that asks
                    # (materialised: a stride-0 view of one sequence's entry is no array)
                    ctx.extras[key] = tuple(t.repeat_interleave(G).contiguous()
                                            for t in (ctx.tok_pos, ctx.tok_seq))
                pos_g, seq_g = ctx.extras[key]
                splits, cluster = ops.decode_plan(ctx.B * G, 1, ctx.max_context, q.device, hd)
                ops.attn_decode(q.view(ctx.B * G, 8 * hd), o.view(ctx.B * G, 8 * hd), kv.k, kv.v,
                                kv.table, pos_g, seq_g, ctx.seq_slot, 8, 1, hd, scale, window,
                                kv.block_tokens, splits, ctx.fault, cluster, sink=sink,
                                bias_near=near, bias_far=far, head_groups=G, bias_slope=tilt)
                return
            # ... else eight at a time
            step = nh if nh // nkv <= 8 else 8
            for h0 in range(0, nh, step):
                n = min(step, nh - h0)
                splits, cluster = ops.decode_plan(ctx.B, nkv, ctx.max_context, q.device, hd)
                ops.attn_decode(q[:, h0 * hd:], o[:, h0 * hd:], kv.k, kv.v, kv.table,
                                ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, n, nkv, hd, scale,
                                window, kv.block_tokens, splits, ctx.fault, cluster,
                                sink=None if sink is None else sink[h0:h0 + n],
                                bias_near=None if near is None else near[h0:h0 + n],
                                bias_far=None if far is None else far[h0:h0 + n],
                                bias_slope=None if tilt is None else tilt[h0:h0 + n])
            return
        if not ctx.is_decode and ops.attn_prefill_supported(hd, kv.block_tokens):
            ops.attn_prefill(q, o, kv.k, kv.v, kv.table, ctx.cu_seqlens, ctx.seq_start,
                             ctx.seq_slot, nh, nkv, hd, scale, window, kv.block_tokens, ctx.B,
                             ctx.max_new, ctx.fault, sink=sink, bias_near=near, bias_far=far,
                             bias_slope=tilt)
            return
    ops.attn_simt(q, o, kv.k, kv.v, kv.table, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                  nh, nkv, hd, scale, window, kv.block_tokens, sink=sink, vd=vd, bias=bias,
                  bias_edges=bias_edges, slope=slope)


@register_part("mixer", "attention")
class Attention(Part):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``window``
    (0 = all keys), ``position`` (a position part's kind and constants), ``names``
    (tensor names of q, k, v, o relative to the layer's prefix).  Optional: ``qk_norm``
    (``{"eps", "q": name, "k": name}``: RMS norm over the whole q and k projections),
    ``values`` (``"keys"``: no value projection, the un-normed keys are the values; needs
    ``qk_norm`` or no position encoding), ``sink`` (name of a [heads] tensor)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.hd = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        self.chunk = int(params.get("chunk") or 0)
        if self.chunk < 0 or self.window < 0 or (self.chunk and self.window):
            raise ValueError("attention: give a sliding `window` or a `chunk`, not both, and "
                             "neither below zero")
        self.mask = -self.chunk if self.chunk else self.window     # as the kernels take it
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads cannot share {self.nkv} key/value heads")
        if not 1 <= self.hd <= 512:
            raise ValueError(f"attention: head_dim {self.hd} is not in [1, 512]; the attention "
                             "kernels take no other head size")
        pos = dict(params.get("position") or {"kind": "none"})
        self.position = build_part("position", PartSpec(pos.pop("kind"), pos), hidden_size,
                                   dtype, device)
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd
        self.qk_norm = params.get("qk_norm")
        self.values_are_keys = params.get("values", "projected") == "keys"
        if params.get("values", "projected") not in ("projected", "keys"):
            raise ValueError(f"attention: values must be 'projected' or 'keys', got "
                             f"{params['values']!r}")
        if self.values_are_keys and self.qk_norm is None:
            raise ValueError("attention: values taken from the keys need qk_norm (the kernel "
                             "that norms the keys stores both)")
        if self.qk_norm is not None and (params.get("position") or {}).get("kind", "none") != "none":
            raise ValueError("attention: qk_norm over the whole projection is built without a "
                             "position encoding only")
        self.sink = None
        # -- the convolved family
        self.vd = int(params.get("value_dim") or self.hd)
        self.o_dim, self.v_dim = self.nh * self.vd, self.nkv * self.vd
        self.own_kv = bool(params.get("own_kv", True))
        self.conv = params.get("conv")
        self.head_norm = params.get("head_norm")
        self.query_gain = params.get("query_gain")
        self.distance_bias = params.get("distance_bias")
        self.bias = self.bias_edges = self.bias_dense = None
        self.bias_names = params.get("bias")
        self.head_gate = params.get("head_gate")
        # the family that norms head by head without a convolution
        self.slope_spec = params.get("distance_slope")
        self.slope = self.slope_log2e = None
        self.headwise = self.conv is None and bool(
            self.bias_names or self.head_gate or self.head_norm or self.vd != self.hd
            or self.chunk or self.slope_spec or not self.own_kv)
        extras = [k for k in ("query_gain", "distance_bias") if params.get(k)] \
            + ([] if self.own_kv or self.headwise else ["own_kv"]) \
            + ([] if self.headwise else
               [k for k in ("head_norm",) if params.get(k)]
               + (["value_dim"] if self.vd != self.hd else []))
        if self.conv is None and extras:
            raise ValueError(f"attention: {extras} are built for convolved projections "
                             "(give `conv`)")
        if self.conv is not None and (self.bias_names or self.head_gate):
            raise ValueError("attention: bias and head_gate are built without a convolution")
        if self.headwise:
            if self.qk_norm is not None or self.values_are_keys:
                raise ValueError("attention: projections normed head by head take no norm over "
                                 "the whole projection and no keys as values")
            if self.head_norm is not None and not (self.head_norm.get("q")
                                                   and self.head_norm.get("k")):
                raise ValueError("attention: head_norm without a convolution names its two "
                                 "weights (q, k)")
            if not 1 <= self.vd <= 512:
                raise ValueError("attention: value_dim must be in [1, 512]")
        if self.conv is not None:
            if self.head_norm is None or self.qk_norm is not None or self.values_are_keys \
                    or (params.get("position") or {}).get("kind", "none") != "none":
                raise ValueError("attention: convolved projections are built with head_norm, "
                                 "without qk_norm, position encoding or keys as values")
            if int(self.conv["taps"]) < 1 or not 1 <= self.vd <= 512:
                raise ValueError("attention: conv.taps must be >= 1 and value_dim in [1, 512]")
            self.taps = int(self.conv["taps"])
            self.conv_channels = self.q_dim + (self.kv_dim + self.v_dim if self.own_kv else 0)
        if params.get("fixed_sink") is not None and params.get("sink"):
            raise ValueError("attention: give `sink` (a tensor) or `fixed_sink`, not both")

    @classmethod
    def weight_specs(cls, params, hidden_size):
        q = params["num_heads"] * params["head_dim"]
        kv = params["num_kv_heads"] * params["head_dim"]
        vdim = params["num_kv_heads"] * (params.get("value_dim") or params["head_dim"])
        o_in = params["num_heads"] * (params.get("value_dim") or params["head_dim"])
        n = params["names"]
        out = {"q": (n["q"], WeightSpec((q, hidden_size))),
               "o": (n["o"], WeightSpec((hidden_size, o_in)))}
        own = params.get("own_kv", True)
        if own:
            out["k"] = (n["k"], WeightSpec((kv, hidden_size)))
        if own and params.get("values", "projected") != "keys":
            out["v"] = (n["v"], WeightSpec((vdim, hidden_size)))
        conv = params.get("conv")
        if conv:
            taps = dict(init=(0.0, 0.5))
            out["q_conv"] = (conv["q"], WeightSpec((q, conv["taps"]), **taps))
            if own:
                out["k_conv"] = (conv["k"], WeightSpec((kv, conv["taps"]), **taps))
                out["v_conv"] = (conv["v"], WeightSpec((vdim, conv["taps"]), **taps))
        if params.get("distance_bias"):
            db = params["distance_bias"]
            out["rel"] = (db["name"], WeightSpec((int(db.get("rows", 64)), params["num_heads"]),
                                                 init=(0.0, 1.0), free=(0,)))
        if params.get("qk_norm"):
            out["q_norm"] = (params["qk_norm"]["q"], WeightSpec((q,), init=(1.0, 0.1)))
            out["k_norm"] = (params["qk_norm"]["k"], WeightSpec((kv,), init=(1.0, 0.1)))
        if params.get("sink"):
            out["sink"] = (params["sink"], WeightSpec((params["num_heads"],), init=(0.0, 1.0)))
        if params.get("bias"):
            b = params["bias"]
            out["q_bias"] = (b["q"], WeightSpec((q,), init=(0.0, 0.1)))
            if own:
                out["k_bias"] = (b["k"], WeightSpec((kv,), init=(0.0, 0.1)))
                out["v_bias"] = (b["v"], WeightSpec((vdim,), init=(0.0, 0.1)))
        hn = params.get("head_norm")
        if hn and not conv and hn.get("q"):
            out["q_head_norm"] = (hn["q"], WeightSpec((params["head_dim"],), init=(1.0, 0.1)))
            out["k_head_norm"] = (hn["k"], WeightSpec((params["head_dim"],), init=(1.0, 0.1)))
        if params.get("head_gate"):
            out["head_gate"] = (params["head_gate"],
                                WeightSpec((params["num_heads"], hidden_size)))
        return out

    def load(self, tensors):
        # one product for q, k and v: rows [q | k | v] of the stacked matrix
        stacked = [tensors["q"]] + ([tensors["k"]] if self.own_kv else []) \
            + ([tensors["v"]] if self.own_kv and not self.values_are_keys else [])
        if self.head_gate:
            stacked.append(tensors["head_gate"])              # rows [q | k | v | gates | zeros]
            self.w_qkv = self._stacked(stacked)
        elif self.headwise:
            self.w_qkv = self._stacked(stacked)               # rows [q | k | v | zeros]
        else:
            self.w_qkv = self._matrix(torch.cat(stacked, dim=0))
        self.in_bias = self.q_head_w = self.k_head_w = None
        if self.bias_names:
            self.in_bias = self._vector32(torch.cat(
                [tensors["q_bias"]] + ([tensors["k_bias"], tensors["v_bias"]]
                                       if self.own_kv else []), dim=0))
        if "q_head_norm" in tensors:
            self.q_head_w = self._vector32(tensors["q_head_norm"])
            self.k_head_w = self._vector32(tensors["k_head_norm"])
        if self.conv is not None:
            taps = [tensors["q_conv"]] + ([tensors["k_conv"], tensors["v_conv"]]
                                          if self.own_kv else [])
            self.conv_w = self._vector32(torch.cat(taps, dim=0))
        if self.distance_bias is not None:
            self.bias = self._vector32(tensors["rel"])
            edges = distance_edges(self.bias.shape[0], float(self.distance_bias["far"]))
            self.bias_edges = torch.from_numpy(edges).to(self.device)
            n_far = int(edges[-1])              # from here on every distance is the last row
            if 1 <= n_far <= FAST_BIAS_MAX_DISTANCES and self.dtype == torch.bfloat16:
                import numpy as np
                row_of = np.searchsorted(edges, np.arange(n_far), side="right") - 1
                log2e = 1.4426950408889634
                near = self.bias[torch.from_numpy(row_of).to(self.device)].t().contiguous()
                self.bias_dense = ((near * log2e).contiguous(),
                                   (self.bias[-1] * log2e).contiguous())
        if self.slope_spec is not None:
            x = float(self.slope_spec["exponent"])
            hs = torch.arange(1, self.nh + 1, dtype=torch.float64)
            slopes = 2.0 ** (-x * hs / self.nh)
            self.slope = self._vector32(slopes)
            self.slope_log2e = self._vector32(slopes * 1.4426950408889634)   # for exp2 kernels
        if self.params.get("fixed_sink") is not None:
            self.sink = torch.full((self.nh,), float(self.params["fixed_sink"]),
                                   dtype=torch.float32, device=self.device)
        self.w_o = self._matrix(tensors["o"])
        if self.qk_norm is not None:
            self.q_norm_w = self._vector32(tensors["q_norm"])
            self.k_norm_w = self._vector32(tensors["k_norm"])
            self.qk_eps = float(self.qk_norm["eps"])
        if "sink" in tensors:
            self.sink = self._vector32(tensors["sink"])
        self.position.load({})

    def prepare(self, max_positions: int) -> None:
        if hasattr(self.position, "prepare"):
            self.position.prepare(max_positions)

    def cache_request(self):
        # (a chunked mask keeps every block: another layer may read these keys with a mask of
        # its own)
        kv = KVRequest(self.nkv, self.hd, self.window,
                       value_dim=0 if self.vd == self.hd else self.vd) if self.own_kv else None
        if self.conv is None or self.taps == 1:
            return kv
        # the last taps - 1 projected rows of every convolved channel
        state = StateRequest((self.conv_channels * (self.taps - 1),), torch.float32)
        return state if kv is None else (kv, state)

    def _forward_convolved(self, x, ctx, cache, into=None):
        """Projections in 32-bit, then one kernel for convolution, head norm, the query's gain
        and the cache write, the saved inputs brought up to date, attention, output product."""
        from .linear import linear_few
        kv = cache.kv
        if kv is None:
            raise ValueError("attention: this layer reads another entry's keys and values, but "
                             "the schedule gives it none")
        proj = linear_few(x, self.w_qkv, out_dtype=torch.float32)
        q = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=x.device)
        gain = self.query_gain or {"coef": 0.0, "every": 0}
        state = cache.state if self.taps > 1 else None
        ops.conv_headnorm_kv_append(
            proj, self.conv_w, state, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_start,
            self.nh, self.nkv if self.own_kv else 0, self.hd, self.vd,
            float(self.head_norm["eps"]), float(gain["coef"]), int(gain["every"]), q,
            table=kv.table, kc=kv.k, vc=kv.v, block_tokens=kv.block_tokens,
            write_cache=cache.writes and self.own_kv, fault=ctx.fault)
        if self.taps > 1:
            ops.delta_conv_state(proj, state, self.taps, self.conv_channels, ctx.cu_seqlens,
                                 ctx.seq_slot, ctx.B)
        o = torch.empty((ctx.T, self.o_dim), dtype=self.dtype, device=x.device)
        self.attend(q, o, ctx, kv)
        if into is not None:
            linear(o, self.w_o, out=into, accumulate=True)
            return None
        return linear_few(o, self.w_o, out_dtype=torch.float32)

    def _forward_headwise(self, x, ctx, cache, into=None, alpha: float = 1.0, proj=None):
        """One product for q|k|v|gates with 32-bit sums (``proj``, where the caller made it
        already), one kernel for bias, head norms, rotation and the cache write, attention, the
        per-head gate, output product."""
        from .linear import linear_few, linear_scaled_add
        kv = cache.kv
        rot = getattr(self.position, "rotary_table", None)
        if rot is not None:
            cos, sin, pairing, rot_dim = rot()
        elif type(self.position).__name__ == "NoPosition":
            cos = sin = None
            pairing = rot_dim = 0
        else:
            raise ValueError("attention: projections normed head by head take a rotary position "
                             "encoding or none")
        proj = linear_few(x, self.w_qkv, out_dtype=torch.float32) if proj is None else proj
        q = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=proj.device)
        if kv is None:
            raise ValueError("attention: this layer reads another entry's keys and values, but "
                             "the schedule gives it none")
        own = self.own_kv
        ops.headnorm_rope_kv_append(
            proj, self.in_bias, self.q_head_w, self.k_head_w,
            float(self.head_norm["eps"]) if self.head_norm else 0.0, cos, sin, pairing, rot_dim,
            ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, self.nh, self.nkv if own else 0, self.hd,
            self.vd, q, table=kv.table, kc=kv.k, vc=kv.v, block_tokens=kv.block_tokens,
            write_cache=cache.writes and own, fault=ctx.fault)
        o = torch.empty((ctx.T, self.o_dim), dtype=self.dtype, device=proj.device)
        self.attend(q, o, ctx, kv)
        if self.head_gate:
            ops.gate_heads(o, proj[:, self.q_dim + (self.kv_dim + self.v_dim if own else 0):],
                           self.nh, self.vd)
        if into is not None:
            linear_scaled_add(o, self.w_o, into, alpha)
            return None
        return linear_few(o, self.w_o, out_dtype=torch.float32)

    @property
    def adds_scaled(self) -> bool:
        """Whether ``forward`` takes ``into`` and ``alpha`` (adds alpha times its output into
        the residual stream itself)."""
        return self.headwise

    def forward(self, x, ctx, cache, into=None, alpha: float = 1.0):
        """``into``: a float32 matrix that the output is added to (the residual stream) instead
        of being returned."""
        from .linear import plain_forced, skinny_max_rows
        if self.headwise:
            return self._forward_headwise(x, ctx, cache, into, alpha)
        if alpha != 1.0:
            raise ValueError("attention: a factor on the output is built for projections normed "
                             "head by head")
        if self.conv is not None:
            return self._forward_convolved(x, ctx, cache, into)
        kv = cache.kv
        rot = getattr(self.position, "rotary_table", None)
        rot = rot() if rot is not None else None         # (cos, sin, pairing, rotary_dim)
        o = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=x.device)
        if self.qk_norm is not None:
            # norms over the whole projections; the kernel that norms the keys stores them
            # (and, when the values are the keys, the un-normed columns as values)
            from .linear import linear_few
            qkv = linear_few(x, self.w_qkv)
            if not self.values_are_keys and cache.writes:
                ops.rope_kv_append(qkv, None, None, 0, 0, self.nh, self.nkv, self.hd,
                                   ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table, kv.k,
                                   kv.v, kv.block_tokens, True, ctx.fault)
            ops.proj_norm_kv_append(qkv, self.q_dim, self.q_norm_w, self.nkv, self.hd,
                                    self.k_norm_w, self.qk_eps, ctx.tok_pos, ctx.tok_seq,
                                    ctx.seq_slot, kv.table, kv.k,
                                    kv.v if self.values_are_keys else None, kv.block_tokens,
                                    cache.writes, ctx.fault)
            self.attend(qkv, o, ctx, kv)
        elif (self.dtype == torch.bfloat16 and ctx.T > skinny_max_rows() and not plain_forced()
                and not _force_plain and self.hd in (64, 128) and rot is not None
                and rot[3] == self.hd and ops.gemm_tc_supported(x, self.w_qkv, o)):
            # many tokens: rotary and the cache write ride in the product's epilogue
            q = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=x.device)
            ops.gemm_tc_qkv_rope(x, self.w_qkv, q, rot[0], rot[1], rot[2], self.nh,
                                 self.nkv, self.hd, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                                 kv.table, kv.k, kv.v, kv.block_tokens, cache.writes)
            self.attend(q, o, ctx, kv)
        else:
            qkv = linear(x, self.w_qkv)                               # [T, q + 2 kv]
            if rot is not None:          # a rotation by table: one kernel encodes and stores
                ops.rope_kv_append(qkv, rot[0], rot[1], rot[2], rot[3], self.nh, self.nkv,
                                   self.hd, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table,
                                   kv.k, kv.v, kv.block_tokens, cache.writes, ctx.fault)
            else:                        # any other encoding, then the store
                self.position.encode(qkv, ctx, self.nh, self.nkv, self.hd)
                if cache.writes:
                    ops.rope_kv_append(qkv, None, None, 0, 0, self.nh, self.nkv, self.hd,
                                       ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table, kv.k,
                                       kv.v, kv.block_tokens, True, ctx.fault)
            self.attend(qkv, o, ctx, kv)
        if into is not None:
            linear(o, self.w_o, out=into, accumulate=True)
            return None
        if self.qk_norm is not None:
            return linear_few(o, self.w_o, out_dtype=torch.float32)
        return linear(o, self.w_o, out_dtype=torch.float32)

    def forward_from_residual(self, h, norm, ctx, cache, alpha: float = 1.0) -> bool:
        """bfloat16.  Few tokens: norm + q|k|v + rotary + cache write in one kernel, attention,
        then the output projection added into ``h``.  Many tokens: the same through the norm's
        kernel and the tensor-core products.  Projections normed head by head: few tokens take
        the input product that norms the rows in its prologue, and ``alpha`` times the output
        product is added into ``h``.  False if the step does not qualify."""
        if norm is not None and self.headwise and self.conv is None:
            from .linear import normed_linear_few
            proj = normed_linear_few(h, norm, self.w_qkv, torch.float32)
            if proj is None:
                return False
            self._forward_headwise(None, ctx, cache, into=h, alpha=alpha, proj=proj)
            return True
        if norm is None or self.conv is not None or self.headwise or alpha != 1.0:
            return False
        if (ctx.T > FUSED_MAX_TOKENS and self.dtype == torch.bfloat16 and not _force_plain
                and h.dtype == torch.float32 and h.is_contiguous()):
            # many tokens: the norm's own kernel, then the products; the last one adds its
            # float32 accumulators into the residual stream, so that no delta is written, read
            # again and added by the next norm
            self.forward(norm.forward(h, None), ctx, cache, into=h)
            return True
        rms = getattr(norm, "rms_params", None)
        rot = getattr(self.position, "rotary_table", None)
        if (_force_plain or not fused_steps_enabled() or self.dtype != torch.bfloat16
                or self.qk_norm is not None or self.sink is not None
                or ctx.T > FUSED_MAX_TOKENS or rms is None or rot is None or cache is None
                or cache.kv is None or cache.kv.block_tokens & (cache.kv.block_tokens - 1)
                or not ops.fused_supported(ctx.T, self.hidden_size, self.w_qkv)
                or not ops.fused_supported(ctx.T, self.q_dim, self.w_o, norm=False)):
            return False
        cos, sin, pairing, rot_dim = rot()
        if rot_dim != self.hd:
            return False
        norm_w, eps = rms()
        kv = cache.kv
        q = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=h.device)
        ops.fused_qkv_rope(h, norm_w, eps, self.w_qkv, q, cos, sin, pairing, self.nh, self.nkv,
                           self.hd, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table, kv.k, kv.v,
                           kv.block_tokens, cache.writes, ctx.fault)
        o = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=h.device)
        self.attend(q, o, ctx, kv)
        ops.fused_linear_add(o, self.w_o, h)
        return True

    def attend(self, q, o, ctx, kv):
        run_attention(q, o, ctx, kv, self.nh, self.nkv, self.hd, self.scale, self.mask,
                      self.dtype, self.sink, vd=self.vd, bias=self.bias,
                      bias_edges=self.bias_edges, bias_dense=self.bias_dense, slope=self.slope,
                      slope_log2e=self.slope_log2e)

    def weight_bytes(self):
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()
