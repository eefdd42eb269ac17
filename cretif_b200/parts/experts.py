"""Routed experts: a feed-forward made of many small gated feed-forwards, of which every token
uses a few.

A router scores the experts per token, ``s = sigmoid(W_router x)`` in 32-bit; the ``top``
experts with the largest scores are chosen and weighted by their scores as they are
(``renormalize`` divides them by their sum).  An expert is ``down(silu(gate x) ⊙ up x)`` without
biases.  ``weight_on`` says where the weight enters: ``"input"`` (the expert sees ``s · x``) or
``"output"`` (its result is scaled).  The output is the sum over the token's experts.

Options: ``gated: False`` makes an expert ``down(act(up x))`` with ``activation`` any of the
kernels' unary activations; ``groups`` (``{"count", "keep"}``) lets the experts form ``count``
equal groups of neighbours, scores a group by the sum of its two largest scores and allows only
experts of the ``keep`` best groups; ``sum_eps`` is added to the sum that ``renormalize`` divides
by; ``shared`` (``{"intermediate_size", "names"}``) is one more expert of the same form that every
token uses with weight one.

The step's (token, choice) pairs are sorted by expert on the device and each expert's rows
are one slice of two grouped products (csrc/moe.cu): gate|up with the activation — and the
weight, when it scales the input: the products are linear, so it is applied to the 32-bit sums —
in its epilogue, then down; the choices are summed in their order.  The grid of every launch is
fixed by the step's size alone, so steps can be captured as CUDA graphs.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from ..config.spec import PartSpec
from .base import Part, build_part, register_part


# Steps of at most this many (token, choice) pairs take the streaming kernel, which reads an
# expert's matrices once per pair; beyond it the pairs are sorted and an expert's rows share a
# tile's read.
FEW_PAIRS = 32
# Steps of more tokens than this compute the router's logits with the library's matrix product
# (in bfloat16 every step does: the few-token product kernels stream the router once).
ROUTE_BY_PRODUCT = 64
_few_pairs_off = False


def few_pairs_off(on=None) -> bool:
    """Switch the few-pairs kernel off (tests run both ways on one step); returns the state."""
    global _few_pairs_off
    if on is not None:
        _few_pairs_off = bool(on)
    return _few_pairs_off


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """params: ``num_experts``, ``top``, ``intermediate_size`` (of one expert), ``weight_on``
    ("input" | "output"), ``renormalize`` (default False), ``names``: ``router`` and the
    patterns ``gate``, ``up``, ``down`` with ``{e}`` for the expert's number.  Optional:
    ``gated`` (default True), ``activation``, ``groups``, ``sum_eps``, ``shared``."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.E = int(params["num_experts"])
        self.top = int(params["top"])
        self.inter = int(params["intermediate_size"])
        self.weight_on = params.get("weight_on", "output")
        self.renorm = bool(params.get("renormalize", False))
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"routed_experts: weight_on must be 'input' or 'output', got "
                             f"{self.weight_on!r}")
        if not 0 < self.top <= self.E or self.E > 256:
            raise ValueError(f"routed_experts: {self.top} of {self.E} experts (at most 256) "
                             "cannot be chosen")
        self.gated = bool(params.get("gated", True))
        self.activation = params.get("activation", "silu")
        if self.gated and self.activation != "silu":
            raise ValueError("routed_experts: gated experts have a kernel for 'silu' only")
        if not self.gated and self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"routed_experts: activation {self.activation!r} has no kernel "
                             f"(there are {sorted(ops.ACTIVATIONS)})")
        groups = params.get("groups") or {}
        self.groups = int(groups.get("count", 0) or 0)
        self.keep = int(groups.get("keep", 0) or 0)
        if self.groups > 1 and (self.E % self.groups or not 1 <= self.keep <= self.groups
                                or self.keep * (self.E // self.groups) < self.top):
            raise ValueError(f"routed_experts: {self.E} experts do not form {self.groups} equal "
                             f"groups of which {self.keep} hold {self.top} experts")
        self.sum_eps = float(params.get("sum_eps", 0.0))
        self.shared = None
        sh = params.get("shared")
        if sh:
            kind = "gated_mlp" if self.gated else "dense_mlp"
            self.shared = build_part("feed_forward", PartSpec(kind, {
                "intermediate_size": int(sh["intermediate_size"]), "activation": self.activation,
                "names": sh["names"]}), hidden_size, dtype, device)

    @classmethod
    def weight_specs(cls, params, hidden_size):
        E, F, n = params["num_experts"], params["intermediate_size"], params["names"]
        out = {"router": (n["router"], WeightSpec((E, hidden_size), init=(0.0, 0.5)))}
        for e in range(E):
            if params.get("gated", True):
                out[f"gate{e}"] = (n["gate"].format(e=e), WeightSpec((F, hidden_size)))
            out[f"up{e}"] = (n["up"].format(e=e), WeightSpec((F, hidden_size)))
            out[f"down{e}"] = (n["down"].format(e=e), WeightSpec((hidden_size, F)))
        sh = params.get("shared")
        if sh:
            Fs, sn = int(sh["intermediate_size"]), sh["names"]
            if params.get("gated", True):
                out["shared_gate"] = (sn["gate"], WeightSpec((Fs, hidden_size)))
            out["shared_up"] = (sn["up"], WeightSpec((Fs, hidden_size)))
            out["shared_down"] = (sn["down"], WeightSpec((hidden_size, Fs)))
        return out

    def load(self, tensors):
        E = self.E
        self.router = self._vector32(tensors["router"])            # 32-bit logits
        # Many tokens: the logits are a matrix product (32-bit sums of exact products) whenever
        # the stored router is exact in the compute type, which a bfloat16 checkpoint's is.
        self.router_matrix = self._matrix(tensors["router"])
        if not torch.equal(self.router_matrix.float(), self.router):
            self.router_matrix = None
        if self.shared is not None:
            self.shared.load({k[len("shared_"):]: v for k, v in tensors.items()
                              if k.startswith("shared_")})
        self.w_down = self._matrix(torch.stack([tensors[f"down{e}"] for e in range(E)]))
        if not self.gated:
            self.w_up = self._matrix(torch.stack([tensors[f"up{e}"] for e in range(E)]))
            return
        # per expert [gate rows | up rows], all experts in one tensor
        self.w_gu = self._matrix(torch.stack(
            [torch.cat([tensors[f"gate{e}"], tensors[f"up{e}"]], dim=0) for e in range(E)]))
        # for the tensor-core grouped product, whose epilogue applies SiLU·mul: gate and up
        # rows of an expert alternate in blocks of 64 (as the dense feed-forward stores them)
        self.w_gu_blocks = None
        F = self.inter
        if self.dtype == torch.bfloat16 and F % 64 == 0 and self.hidden_size % 8 == 0:
            self.w_gu_blocks = self._matrix(torch.stack([torch.stack(
                [tensors[f"gate{e}"].reshape(F // 64, 64, -1),
                 tensors[f"up{e}"].reshape(F // 64, 64, -1)], dim=1).reshape(2 * F, -1)
                for e in range(E)]))

    def forward(self, x, ctx):
        T, H = x.shape
        dev = x.device
        P = T * self.top
        ids = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        wts = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        if self.router_matrix is not None and (T > ROUTE_BY_PRODUCT
                                               or self.dtype == torch.bfloat16):
            from .linear import linear_few
            logits = linear_few(x, self.router_matrix, out_dtype=torch.float32)
            ops.moe_topk(logits, self.top, ids, wts, renorm=self.renorm, groups=self.groups,
                         keep=self.keep, sum_eps=self.sum_eps)
        else:
            ops.moe_route(x, self.router, self.top, ids, wts, renorm=self.renorm,
                          groups=self.groups, keep=self.keep, sum_eps=self.sum_eps)
        y = torch.empty((T, H), dtype=torch.float32, device=dev)
        if self.gated:
            self._gated_experts(x, ids, wts, y)
        else:
            self._plain_experts(x, ids, wts, y)
        if self.shared is not None:
            self.shared.forward(x, ctx, into=y)
        return y

    def _plain_experts(self, x, ids, wts, y):
        """Experts without a gate: the activation sits in the first product's epilogue."""
        T, H = x.shape
        dev, P = x.device, T * self.top
        on_input = self.weight_on == "input"
        mode = ops.moe_act_mode(self.activation)
        if P <= FEW_PAIRS and not few_pairs_off():
            act = torch.empty((P, self.inter), dtype=self.dtype, device=dev)
            rows = torch.empty((P, H), dtype=torch.float32, device=dev)
            ops.moe_gemv(x, self.w_up, act, self.top, mode, 1 if on_input else 0, ids, wts)
            ops.moe_gemv(act, self.w_down, rows, self.top, 1, 0 if on_input else 2, ids, wts)
            ops.moe_combine(rows, None, self.top, y)
            return
        if self.dtype == torch.bfloat16 and ops.moe_tc_supported(x, self.w_up, self.w_down,
                                                                 gated=False):
            tiles = ops.moe_tc_tiles(P, self.E)
            idx = torch.empty(P + tiles + 1, dtype=torch.int32, device=dev)
            place, tile_expert, used = idx[:P], idx[P:P + tiles], idx[P + tiles:]
            ops.moe_group_padded(ids, self.E, place, tile_expert, used)
            rows_pad = tiles * ops.MOE_TC_TILE
            xs = torch.empty((rows_pad, H), dtype=self.dtype, device=dev)
            ops.moe_gather_rows(x, xs, place, wts if on_input else None, self.top)
            act = torch.empty((rows_pad, self.inter), dtype=self.dtype, device=dev)
            ops.gemm_tc_act_grouped(xs, self.w_up, act, tile_expert, used, self.activation)
            rows = torch.empty((rows_pad, H), dtype=torch.float32, device=dev)
            ops.gemm_tc_grouped(act, self.w_down, rows, tile_expert, used)
            ops.moe_combine(rows, place, self.top, y, wts=None if on_input else wts)
            return
        tiles = ops.moe_max_tiles(P, self.E)
        idx = torch.empty(self.E + 1 + 2 * P + 2 * tiles, dtype=torch.int32, device=dev)
        offsets, place, order = idx[:self.E + 1], idx[self.E + 1:self.E + 1 + P], \
            idx[self.E + 1 + P:self.E + 1 + 2 * P]
        tile_expert, tile_row0 = idx[self.E + 1 + 2 * P:self.E + 1 + 2 * P + tiles], \
            idx[self.E + 1 + 2 * P + tiles:]
        ops.moe_group(ids, self.E, offsets, place, order, tile_expert, tile_row0)
        act = torch.empty((P, self.inter), dtype=self.dtype, device=dev)
        rows = torch.empty((P, H), dtype=torch.float32, device=dev)
        ops.moe_gemm(x, self.w_up, act, self.top, mode, 1 if on_input else 0, wts, order, offsets,
                     tile_expert, tile_row0)
        ops.moe_gemm(act, self.w_down, rows, self.top, 1, 0 if on_input else 2, wts, order,
                     offsets, tile_expert, tile_row0)
        ops.moe_combine(rows, place, self.top, y)

    def _gated_experts(self, x, ids, wts, y):
        T, H = x.shape
        dev, P = x.device, T * self.top
        on_input = self.weight_on == "input"
        if P <= FEW_PAIRS and not few_pairs_off():
            # a handful of pairs: every pair streams its expert's rows, nothing is sorted
            act = torch.empty((P, self.inter), dtype=self.dtype, device=dev)
            rows = torch.empty((P, H), dtype=torch.float32, device=dev)
            ops.moe_gemv(x, self.w_gu, act, self.top, 0, 1 if on_input else 0, ids, wts)
            ops.moe_gemv(act, self.w_down, rows, self.top, 1, 0 if on_input else 2, ids, wts)
            ops.moe_combine(rows, None, self.top, y)
            return
        if self.w_gu_blocks is not None and ops.moe_tc_supported(x, self.w_gu_blocks, self.w_down):
            # many pairs, bfloat16: the tcgen05 product in its grouped mode over rows sorted
            # into whole 128-row tiles per expert; the router weight goes into the gathered rows
            tiles = ops.moe_tc_tiles(P, self.E)
            idx = torch.empty(P + tiles + 1, dtype=torch.int32, device=dev)
            place, tile_expert, used = idx[:P], idx[P:P + tiles], idx[P + tiles:]
            ops.moe_group_padded(ids, self.E, place, tile_expert, used)
            rows_pad = tiles * ops.MOE_TC_TILE
            xs = torch.empty((rows_pad, H), dtype=self.dtype, device=dev)
            ops.moe_gather_rows(x, xs, place, wts if on_input else None, self.top)
            act = torch.empty((rows_pad, self.inter), dtype=self.dtype, device=dev)
            ops.gemm_tc_silu_grouped(xs, self.w_gu_blocks, act, tile_expert, used)
            rows = torch.empty((rows_pad, H), dtype=torch.float32, device=dev)
            ops.gemm_tc_grouped(act, self.w_down, rows, tile_expert, used)
            ops.moe_combine(rows, place, self.top, y, wts=None if on_input else wts)
            return
        tiles = ops.moe_max_tiles(P, self.E)
        idx = torch.empty(self.E + 1 + 2 * P + 2 * tiles, dtype=torch.int32, device=dev)
        offsets, place, order = idx[:self.E + 1], idx[self.E + 1:self.E + 1 + P], \
            idx[self.E + 1 + P:self.E + 1 + 2 * P]
        tile_expert, tile_row0 = idx[self.E + 1 + 2 * P:self.E + 1 + 2 * P + tiles], \
            idx[self.E + 1 + 2 * P + tiles:]
        ops.moe_group(ids, self.E, offsets, place, order, tile_expert, tile_row0)
        act = torch.empty((P, self.inter), dtype=self.dtype, device=dev)
        rows = torch.empty((P, H), dtype=torch.float32, device=dev)
        ops.moe_gemm(x, self.w_gu, act, self.top, 0, 1 if on_input else 0, wts, order, offsets,
                     tile_expert, tile_row0)
        ops.moe_gemm(act, self.w_down, rows, self.top, 1, 0 if on_input else 2, wts, order,
                     offsets, tile_expert, tile_row0)
        ops.moe_combine(rows, place, self.top, y)

    def weight_bytes(self):
        # (the blocked copy of gate|up serves the many-pairs path and is not counted twice)
        first = self.w_gu if self.gated else self.w_up
        return ((first.numel() + self.w_down.numel()) * self.w_down.element_size()
                + 4 * self.router.numel()
                + (self.shared.weight_bytes() if self.shared is not None else 0))
