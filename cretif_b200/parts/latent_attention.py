"""Attention over a cached low-rank latent, with a sliding window and a softmax sink.

Per token the layer projects queries ``q = W_q x`` (heads × dim) and a latent
``c = rmsnorm(W_down x)`` of ``latent_rank`` numbers; head h's keys and values are
``k = W_uk[h] c`` and ``v = W_uv[h] c``.  Only ``c`` is cached.  The kernels never expand it:

    score  = q_h · (W_uk[h] c) = (W_uk[h]ᵀ q_h) · c        -> the query is moved into latent space
    out_h  = Σ p (W_uv[h] c)   = W_uv[h] (Σ p c)           -> the values are expanded once, after

so the attention itself is multi-query attention with ONE key/value head of size
``latent_rank`` whose keys and values are the same cached rows, and every attention kernel
of the library serves it as it is.  The two per-head products around it are one batched launch
each.  The softmax's denominator may hold one more term ``exp(sink_h)`` per head, unscaled, with
no key and no value.

Options beyond that: the queries may pass a latent of their own, ``q = W_uq rmsnorm(W_dq x)``
(``q_rank``); a position encoding may rotate a part of every query head and ONE extra key part
that all heads share (``rot_dim`` with ``position``): a query head is ``[flat (head_dim) |
rotated (rot_dim)]``, the down projection has ``latent_rank + rot_dim`` rows of which the last
``rot_dim`` are that key part (not normed), and the score is the sum of both dot products.  The
cached row is then ``[c | rotated key part]``, the query in latent space
``[W_uk[h]ᵀ q_flat | q_rotated]``: still one key/value head, of size ``latent_rank + rot_dim``,
whose first ``latent_rank`` output columns are the ones the values are expanded from.  An output
gate ``sigmoid(W_g x)`` multiplies the heads' outputs channel by channel (``gate: "channel"``) or
head by head (``gate: "head"``) before the output projection.
"""
from __future__ import annotations

import torch

from ..cache import KVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from .attention import run_attention
from .base import Part, build_part, register_part
from .linear import linear_few as linear


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: ``num_heads``, ``head_dim`` (query/key size per head), ``value_dim``,
    ``latent_rank``, ``scale``, ``window`` (0 = all keys), ``eps`` (of the latent's norm),
    ``names`` (q, down, down_norm, up_k, up_v, o and, optionally, sink).  Optional: ``q_rank``
    (the queries' latent; names q_down, q_norm, q_up instead of q), ``rot_dim`` with ``position``
    (a rotary position part's constants; its ``rotary_dim``, by default all of ``rot_dim``, says
    how many of the rotated part's first channels turn), ``gate`` ("channel" | "head", name
    ``gate``)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.hd = int(params["head_dim"])
        self.vd = int(params["value_dim"])
        self.rank = int(params["latent_rank"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        self.eps = float(params["eps"])
        if min(self.nh, self.hd, self.vd, self.rank) <= 0:
            raise ValueError("latent_attention: sizes must be positive")
        self.q_rank = int(params.get("q_rank") or 0)
        self.rot = int(params.get("rot_dim") or 0)
        self.gate = params.get("gate")
        self.key_dim = self.rank + self.rot            # the one cached head
        if self.key_dim > 512:
            raise ValueError(f"latent_attention: latent_rank + rot_dim = {self.key_dim} is above "
                             "512; the attention kernels take no larger head")
        if self.gate not in (None, "channel", "head"):
            raise ValueError(f"latent_attention: gate must be 'channel' or 'head', got "
                             f"{self.gate!r}")
        self.extended = bool(self.q_rank or self.rot or self.gate)
        if self.extended and not self.q_rank:
            raise ValueError("latent_attention: a rotated part and an output gate are built for "
                             "queries that pass a latent (give q_rank)")
        self.position = None
        if self.rot:
            pos = dict(params.get("position") or {})
            if pos.pop("kind", "rotary") != "rotary" or self.rot % 2:
                raise ValueError("latent_attention: the rotated part takes a rotary position "
                                 "encoding of an even size")
            pos["rotary_dim"] = int(pos.get("rotary_dim") or self.rot)
            if not 0 < pos["rotary_dim"] <= self.rot or pos["rotary_dim"] % 2:
                raise ValueError("latent_attention: the rotation takes an even number of the "
                                 "rotated part's channels")
            self.position = build_part("position", PartSpec("rotary", pos), hidden_size, dtype,
                                       device)
        self.sink = None

    @classmethod
    def weight_specs(cls, params, hidden_size):
        H, d, e, r = (params["num_heads"], params["head_dim"], params["value_dim"],
                      params["latent_rank"])
        n = params["names"]
        qr, rot = int(params.get("q_rank") or 0), int(params.get("rot_dim") or 0)
        out = {"down": (n["down"], WeightSpec((r + rot, hidden_size))),
               "down_norm": (n["down_norm"], WeightSpec((r,), init=(1.0, 0.1))),
               "up_k": (n["up_k"], WeightSpec((H * d, r))),
               "up_v": (n["up_v"], WeightSpec((H * e, r))),
               "o": (n["o"], WeightSpec((hidden_size, H * e)))}
        if qr:
            out["q_down"] = (n["q_down"], WeightSpec((qr, hidden_size)))
            out["q_norm"] = (n["q_norm"], WeightSpec((qr,), init=(1.0, 0.1)))
            out["q_up"] = (n["q_up"], WeightSpec((H * (d + rot), qr)))
        else:
            out["q"] = (n["q"], WeightSpec((H * d, hidden_size)))
        if params.get("gate"):
            rows = H * e if params["gate"] == "channel" else H
            out["gate"] = (n["gate"], WeightSpec((rows, hidden_size)))
        if n.get("sink"):
            out["sink"] = (n["sink"], WeightSpec((H,), init=(0.0, 1.0)))
        return out

    def load(self, tensors):
        H, d, e, r = self.nh, self.hd, self.vd, self.rank
        if self.extended:
            # one product for [cq | c | rotated key part | gates], 32-bit sums
            self.w_in = self._stacked([tensors["q_down"], tensors["down"]]
                                      + ([tensors["gate"]] if self.gate else []))
            self.w_q_up = self._matrix(tensors["q_up"])
            self.q_norm = self._vector32(tensors["q_norm"])
            if self.position is not None:
                self.position.load({})
        else:
            self.w_in = self._matrix(torch.cat([tensors["q"], tensors["down"]], dim=0))  # [q | c]
        # W_uk[h] is [d, r]; the query goes to latent space through its transpose [r, d]
        self.w_q_latent = self._matrix(tensors["up_k"].reshape(H, d, r).transpose(1, 2))
        self.w_up_v = self._matrix(tensors["up_v"].reshape(H, e, r))
        self.w_o = self._matrix(tensors["o"])
        self.down_norm = self._vector32(tensors["down_norm"])
        if "sink" in tensors:
            self.sink = self._vector32(tensors["sink"])

    def prepare(self, max_positions: int) -> None:
        if self.position is not None:
            self.position.prepare(max_positions)

    def cache_request(self):
        return KVRequest(1, self.key_dim, self.window, shared_values=True)

    def _forward_extended(self, x, ctx, cache, into=None, proj=None):
        """The queries through their latent, a rotated part beside the latent, an output gate.
        ``proj``: the input product's 32-bit result, where the caller made it already."""
        H, d, e, r, rot, T, D = self.nh, self.hd, self.vd, self.rank, self.rot, ctx.T, self.key_dim
        kv = cache.kv
        cos = sin = None
        pairing = rdims = 0
        if self.position is not None:
            cos, sin, pairing, rdims = self.position.rotary_table()
        if proj is None:
            proj = linear(x, self.w_in, out_dtype=torch.float32)    # [cq | c | kr | gates | 0]
        dev = proj.device
        cq = torch.empty((T, self.q_rank), dtype=self.dtype, device=dev)
        ops.latent_in(proj, self.q_rank, r, rot, self.q_norm, self.down_norm, self.eps, cos, sin,
                      pairing, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, cq, table=kv.table,
                      kc=kv.k, block_tokens=kv.block_tokens, write_cache=cache.writes,
                      fault=ctx.fault, rot_dims=rdims)
        q = linear(cq, self.w_q_up)                                   # [T, H (d + rot)]
        q_lat = torch.empty((T, H, D), dtype=self.dtype, device=dev)
        ops.gemm_batched(q.view(T, H, d + rot)[:, :, :d], self.w_q_latent, q_lat[:, :, :r])
        ops.rope_heads(q, H, d, rot, cos, sin, pairing, ctx.tok_pos, q_lat, r, rot_dims=rdims)
        o_lat = torch.empty((T, H * D), dtype=self.dtype, device=dev)
        run_attention(q_lat.view(T, H * D), o_lat, ctx, kv, H, 1, D, self.scale, self.window,
                      self.dtype, self.sink)
        o = torch.empty((T, H, e), dtype=self.dtype, device=dev)
        ops.gemm_batched(o_lat.view(T, H, D)[:, :, :r], self.w_up_v, o)
        o = o.view(T, H * e)
        if self.gate:
            gates = proj[:, self.q_rank + r + rot:]
            if self.gate == "channel":
                ops.gate_heads(o, gates, H * e, 1)
            else:
                ops.gate_heads(o, gates, H, e)
        if into is not None:
            linear(o, self.w_o, out=into, accumulate=True)
            return None
        return linear(o, self.w_o, out_dtype=torch.float32)

    def forward(self, x, ctx, cache, into=None):
        """``into``: a float32 matrix that the output is added to (the residual stream) instead
        of being returned."""
        if self.extended:
            return self._forward_extended(x, ctx, cache, into)
        H, d, e, r, T = self.nh, self.hd, self.vd, self.rank, ctx.T
        kv = cache.kv
        qc = linear(x, self.w_in)                                   # [T, H d + r]
        # the latent is normed and stored as the one key/value head; q is left as it is
        ops.proj_norm_kv_append(qc, H * d, None, 1, r, self.down_norm, self.eps, ctx.tok_pos,
                                ctx.tok_seq, ctx.seq_slot, kv.table, kv.k, None, kv.block_tokens,
                                cache.writes, ctx.fault)
        q_lat = torch.empty((T, H, r), dtype=self.dtype, device=x.device)
        ops.gemm_batched(qc[:, :H * d].unflatten(1, (H, d)), self.w_q_latent, q_lat)
        o_lat = torch.empty((T, H * r), dtype=self.dtype, device=x.device)
        run_attention(q_lat.view(T, H * r), o_lat, ctx, kv, H, 1, r, self.scale, self.window,
                      self.dtype, self.sink)
        o = torch.empty((T, H, e), dtype=self.dtype, device=x.device)
        ops.gemm_batched(o_lat.view(T, H, r), self.w_up_v, o)
        if into is not None:
            linear(o.view(T, H * e), self.w_o, out=into, accumulate=True)
            return None
        return linear(o.view(T, H * e), self.w_o, out_dtype=torch.float32)

    def forward_from_residual(self, h, norm, ctx, cache) -> bool:
        """The output product is added into ``h``.  Few tokens in bfloat16: the block's norm runs
        in the prologue of the input product; else the norm has a kernel of its own."""
        if norm is None or h.dtype != torch.float32 or not h.is_contiguous():
            return False
        if self.extended and self.dtype == torch.bfloat16:
            from .linear import normed_linear_few
            proj = normed_linear_few(h, norm, self.w_in, torch.float32)
            if proj is not None:
                self._forward_extended(None, ctx, cache, into=h, proj=proj)
                return True
        self.forward(norm.forward(h, None), ctx, cache, into=h)
        return True

    def weight_bytes(self):
        n = (self.w_in.numel() + self.w_q_latent.numel() + self.w_up_v.numel()
             + self.w_o.numel() + (self.w_q_up.numel() if self.extended else 0))
        return n * self.w_o.element_size()
