"""Token embedding and the output head.

The embedding gathers rows of ``[vocab, hidden]`` without scaling
(src/embedding.cu:39-60) into the 32-bit residual stream; the head multiplies the
normed rows that were asked for by ``[vocab, hidden]ᵀ`` (src/embedding.cu:85-135),
sharing the embedding matrix when the model ties them (src/model.cu:1024-1039).
The reference computes logits for every row of a step; the head here only sees the
rows whose logits are wanted.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """params: ``name``; sized by the model's vocabulary (``vocab_size`` is injected).
    Optional ``positions`` (``{"name", "rows"}``): a learned vector per position, a table of
    ``rows`` positions, added to the token's row as it is (32-bit sum).  Optional ``norm``
    (``{"name", "eps", "offset"}``): an RMS norm of the gathered row, its weight stored as the
    factor minus ``offset``, in 32-bit, before the first layer reads the stream."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        out = {"table": (params["name"], WeightSpec((params["vocab_size"], hidden_size)))}
        pos = params.get("positions")
        if pos:
            out["positions"] = (pos["name"], WeightSpec((int(pos["rows"]), hidden_size)))
        norm = params.get("norm")
        if norm:
            mean = 1.0 - float(norm.get("offset", 0.0))
            out["norm"] = (norm["name"], WeightSpec((hidden_size,), init=(mean, 0.02)))
        return out

    def load(self, tensors):
        self.table = self._matrix(tensors["table"])
        self.positions = self._matrix(tensors["positions"]) if "positions" in tensors else None
        self.norm_weight = None
        if "norm" in tensors:
            spec = self.params["norm"]
            self.norm_weight = (self._vector32(tensors["norm"])
                                + float(spec.get("offset", 0.0))).contiguous()
            self.norm_eps = float(spec["eps"])

    def prepare(self, max_positions: int) -> None:
        if self.positions is not None and max_positions > self.positions.shape[0]:
            raise ValueError(f"the model has {self.positions.shape[0]} learned positions; "
                             f"sequences of up to {max_positions} tokens were asked for")

    def forward(self, ids, ctx):
        h = torch.empty((ids.numel(), self.hidden_size), dtype=torch.float32, device=ids.device)
        ops.embed_rows(self.table, ids, h, ctx.fault, positions=self.positions,
                       tok_pos=ctx.tok_pos if self.positions is not None else None)
        if self.norm_weight is not None:
            ops.rmsnorm_rows(h, self.norm_weight, self.norm_eps)
        return h

    def weight_bytes(self):
        n = self.table.numel() + (self.positions.numel() if self.positions is not None else 0)
        return n * self.table.element_size() + (4 * self.hidden_size
                                                if self.norm_weight is not None else 0)


@register_part("head", "linear_head")
class LinearHead(Part):
    """params: ``tied`` (share the embedding matrix), ``name``, ``vocab_size``; optional
    ``softcap`` c: the logits leave as ``c * tanh(logits / c)``."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        if params.get("tied"):
            return {}
        return {"weight": (params["name"], WeightSpec((params["vocab_size"], hidden_size)))}

    def load(self, tensors):
        self.weight = None if self.params.get("tied") else self._matrix(tensors["weight"])

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.table

    def _capped(self, logits):
        cap = self.params.get("softcap")
        if cap and logits.numel():
            ops.softcap(logits, float(cap))
        return logits

    def forward(self, n, ctx):
        return self._capped(linear(n, self.weight, out_dtype=torch.float32))

    def forward_from_residual(self, h, pending, norm, rows, ctx):
        """Few wanted rows, bfloat16: final norm and head product in one kernel; None if the
        step does not qualify."""
        from .attention import FUSED_MAX_TOKENS, fused_steps_enabled
        R = h.shape[0] if rows is None else rows.numel()
        rms = getattr(norm, "rms_params", None)
        if (pending is not None or not fused_steps_enabled() or self.dtype != torch.bfloat16
                or R > FUSED_MAX_TOKENS or rms is None
                or not ops.fused_supported(R, self.hidden_size, self.weight)):
            return None
        logits = torch.empty((R, self.weight.shape[0]), dtype=torch.float32, device=h.device)
        norm_w, eps = rms()
        ops.fused_norm_linear(h, norm_w, eps, self.weight, logits, rows=rows)
        return self._capped(logits)

    def weight_bytes(self):
        if self.params.get("tied") or self.weight is None:
            return 0
        return self.weight.numel() * self.weight.element_size()
