"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

Per token, with ``x`` the mixer's input: ``q = W_q x`` and ``k = W_k x`` (heads × dim),
``v = W_v x`` (heads × value_dim), no biases.  q and k are position-encoded (a rotation of the
first channels of every head), then k is multiplied by ``dim^-1/2``.  Head h keeps a matrix
``S`` [dim, value_dim] with a constant decay ``g_h`` in (0, 1]:

    S <- g_h S + k vᵀ;   o = Sᵀ q

``o`` is divided by its root mean square per head (no weight), the heads are concatenated,
multiplied by ``silu(W_g x)`` and projected by ``W_o``.  Between steps a sequence keeps S in
32-bit: one fixed-size state per cache slot, zeroed when the slot is handed out.  The four
projections are one product whose result stays in 32-bit, as does everything after it up to
the normed, gated output.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, build_part, register_part
from .linear import linear_few, linear_scaled_add, normed_linear_few


@register_part("mixer", "retention")
class Retention(Part):
    """params: ``num_heads``, ``head_dim``, ``value_dim`` (default head_dim), ``decay`` (a
    number per head), ``eps`` (of the output norm), ``position`` (a position part's kind and
    constants: rotary or none), ``key_scale`` (default head_dim^-1/2), ``names`` (q, k, v,
    gate, o)."""

    graph_safe = True
    adds_scaled = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.hd = int(params["head_dim"])
        self.vd = int(params.get("value_dim") or self.hd)
        self.eps = float(params["eps"])
        decay = [float(g) for g in params["decay"]]
        if min(self.nh, self.hd, self.vd) <= 0 or len(decay) != self.nh:
            raise ValueError(f"retention: sizes must be positive and {self.nh} heads need "
                             f"{self.nh} decays, got {len(decay)}")
        if self.hd > 1024:
            raise ValueError(f"retention: head_dim {self.hd} exceeds 1024 (a column's rows stay "
                             "in one warp's registers)")
        self.decay_host = decay
        self.key_scale = float(params.get("key_scale", self.hd ** -0.5))
        pos = dict(params.get("position") or {"kind": "none"})
        self.position = build_part("position", PartSpec(pos.pop("kind"), pos), hidden_size,
                                   dtype, device)
        self.state_floats = self.nh * self.hd * self.vd

    @classmethod
    def weight_specs(cls, params, hidden_size):
        H, d = params["num_heads"], params["head_dim"]
        e = params.get("value_dim") or d
        n = params["names"]
        return {"q": (n["q"], WeightSpec((H * d, hidden_size))),
                "k": (n["k"], WeightSpec((H * d, hidden_size))),
                "v": (n["v"], WeightSpec((H * e, hidden_size))),
                "gate": (n["gate"], WeightSpec((H * e, hidden_size))),
                "o": (n["o"], WeightSpec((hidden_size, H * e)))}

    def load(self, tensors):
        t = tensors
        # one product: [q | k | v | gate]
        self.w_in = self._stacked([t["q"], t["k"], t["v"], t["gate"]])
        self.w_o = self._matrix(t["o"])
        self.decay = torch.tensor(self.decay_host, dtype=torch.float32, device=self.device)
        self.position.load({})

    def prepare(self, max_positions: int) -> None:
        if hasattr(self.position, "prepare"):
            self.position.prepare(max_positions)

    def cache_request(self):
        return StateRequest((self.state_floats,), torch.float32)

    def forward(self, x, ctx, cache, into=None, alpha: float = 1.0):
        """``into``: a float32 matrix that ``alpha`` times the output is added to (the residual
        stream) instead of the output being returned."""
        proj = linear_few(x, self.w_in, out_dtype=torch.float32)      # [T, 2Hd + 2He (+ pad)]
        return self._finish(proj, ctx, cache, into, alpha)

    def forward_from_residual(self, h, norm, ctx, cache, alpha: float = 1.0) -> bool:
        """Few tokens in bfloat16: the norm runs in the input product's prologue and the output
        product adds ``alpha`` times its sums into ``h``.  False if the step does not qualify."""
        proj = normed_linear_few(h, norm, self.w_in, torch.float32)
        if proj is None:
            return False
        self._finish(proj, ctx, cache, h, alpha)
        return True

    def _finish(self, proj, ctx, cache, into, alpha):
        H, d, e = self.nh, self.hd, self.vd
        T = ctx.T
        rot = getattr(self.position, "rotary_table", None)
        if rot is not None:
            cos, sin, pairing, rot_dim = rot()
        elif type(self.position).__name__ == "NoPosition":
            cos = sin = None
            pairing = rot_dim = 0
        else:
            raise ValueError("retention takes a rotary position encoding or none")
        prep = torch.empty((T, 2 * H * d), dtype=torch.float32, device=proj.device)
        ops.retention_prepare(proj, prep, cos, sin, pairing, rot_dim, ctx.tok_pos, H, d,
                              self.key_scale)
        o_raw = torch.empty((T, H * e), dtype=torch.float32, device=proj.device)
        ops.retention_recurrence(prep, proj[:, 2 * H * d:2 * H * d + H * e], self.decay,
                                 cache.state, ctx.cu_seqlens, ctx.seq_slot, ctx.B, H, d, e,
                                 o_raw, write_state=cache.writes)
        out = torch.empty((T, H * e), dtype=self.dtype, device=proj.device)
        ops.heads_out_norm(o_raw, proj[:, 2 * H * d + H * e:2 * H * d + 2 * H * e], None,
                           self.eps, out, H, e)
        if into is not None:
            linear_scaled_add(out, self.w_o, into, alpha)
            return None
        return linear_few(out, self.w_o, out_dtype=torch.float32)

    def weight_bytes(self):
        return (self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size() + 4 * self.nh
