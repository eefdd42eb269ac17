"""Matrix products ``y = x · Wᵀ`` for the parts, with the choice of kernel in one place.

``W`` is stored ``[out, in]`` as in the checkpoint (K-major, which is what every
kernel here wants), ``x`` is ``[tokens, in]``.  The reference dispatches on the
weight format (``matmul_dispatch``, src/model.cu:797-825); here the choice is by
compute dtype and by the number of rows:

* float32: the CUDA-core FMA kernel, always (true 32-bit arithmetic);
* bfloat16, few rows (decode): the weight-streaming kernel;
* bfloat16, many rows (prefill): the tcgen05 tensor-core kernel;
* any shape a fast kernel refuses (alignment, size) goes to the CUDA-core kernel,
  which takes every shape.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops

# Rows up to which the weight-streaming kernel is used instead of the tensor-core one.
SKINNY_MAX_ROWS = 32

_force_plain = False


def force_plain_kernels(on: bool) -> None:
    """Route every product to the CUDA-core kernel (used by tests as the yardstick)."""
    global _force_plain
    _force_plain = bool(on)


def plain_forced() -> bool:
    return _force_plain


def skinny_max_rows() -> int:
    return SKINNY_MAX_ROWS


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and not _force_plain:
        if M <= SKINNY_MAX_ROWS and ops.gemv_supported(x, w, out):
            ops.gemv_bf16(x, w, out, accumulate)
            return out
        if ops.gemm_tc_supported(x, w, out):
            ops.gemm_tc(x, w, out, accumulate)
            return out
    ops.gemm_simt(x, w, out, accumulate)
    return out


FEW_ROWS = 64


def _few_rows(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the few-token kernels take this product."""
    from .attention import fused_steps_enabled
    M, K = x.shape
    return (0 < M <= FEW_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and not _force_plain and fused_steps_enabled() and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and ops.fused_supported(M, K, w, norm=False))


def linear_few(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``linear`` for parts that read rows which are already in the compute type: bfloat16
    steps of at most 64 rows take the few-token kernels (weights streamed once through shared
    memory or registers, launched as programmatic dependents), everything else ``linear``."""
    M, K = x.shape
    if _few_rows(x, w):
        if out is None:
            out = torch.empty((M, w.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
        if out.dtype == torch.float32 or not accumulate:
            ops.fused_linear_x(x, w, out, accumulate)
            return out
    return linear(x, w, out_dtype=out_dtype, out=out, accumulate=accumulate)


def normed_linear_few(h: torch.Tensor, norm, w: torch.Tensor, out_dtype,
                      unary: Optional[str] = None) -> Optional[torch.Tensor]:
    """``[act](rmsnorm(h) · Wᵀ)`` by the few-token kernel that norms the residual rows in its
    own prologue (and rounds them to bfloat16 as the norm's kernel would), or None where the
    step, the norm or the sizes do not allow it."""
    from .attention import fused_steps_enabled
    rms = getattr(norm, "rms_params", None)
    M, K = h.shape
    if (rms is None or not 0 < M <= FEW_ROWS or w.dtype != torch.bfloat16 or _force_plain
            or not fused_steps_enabled() or h.dtype != torch.float32 or not h.is_contiguous()
            or not ops.fused_supported(M, K, w)):
        return None
    norm_w, eps = rms()
    out = torch.empty((M, w.shape[0]), dtype=out_dtype, device=h.device)
    ops.fused_norm_linear(h, norm_w, eps, w, out, unary=unary)
    return out


def linear_scaled_add(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, alpha: float) -> None:
    """``h += alpha * x · Wᵀ`` with ``h`` a float32 matrix (the residual stream).  With
    ``alpha`` 1 the product's kernels add their 32-bit sums into ``h`` themselves; with any other
    factor the tensor-core product and the few-token kernels scale their sums before they add
    them, and the other kernels go through a 32-bit product and one fused multiply-add per
    element."""
    if alpha == 1.0:
        linear_few(x, w, out=h, accumulate=True)
        return
    if (x.shape[0] > FEW_ROWS and x.dtype == torch.bfloat16 and not _force_plain
            and ops.gemm_tc_supported(x, w, h)):
        ops.gemm_tc(x, w, h, accumulate=True, alpha=float(alpha))   # scaled in the epilogue
        return
    if _few_rows(x, w):
        ops.fused_linear_x(x, w, h, accumulate=True, alpha=float(alpha))
        return
    y = linear_few(x, w, out_dtype=torch.float32)
    ops.axpy_rows(h, y, float(alpha))


def linear_activation(x: torch.Tensor, w: torch.Tensor, kind: str, dtype) -> torch.Tensor:
    """``act(x · Wᵀ)`` in ``dtype``, the activation on the product's 32-bit sums: in the
    epilogue of the tensor-core product or of the few-token kernels where they take the step,
    else as a kernel of its own over a 32-bit result."""
    M = x.shape[0]
    act = torch.empty((M, w.shape[0]), dtype=dtype, device=x.device)
    if (M > FEW_ROWS and x.dtype == torch.bfloat16 and not _force_plain
            and ops.gemm_tc_supported(x, w, act)):
        ops.gemm_tc(x, w, act, unary=kind)
        return act
    if act.dtype == torch.bfloat16 and _few_rows(x, w):
        ops.fused_linear_x(x, w, act, unary=kind)
        return act
    up = linear_few(x, w, out_dtype=torch.float32)
    ops.activation(up, act, kind)
    return act
