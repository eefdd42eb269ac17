"""Python faces of the CUDA launchers: argument checks, then one ctypes call each.

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, sizes) and raises ``KernelError`` with a plain message when a kernel
refuses its arguments.  There is no fallback of any kind: without the compiled
library, or with a tensor that is not on a CUDA device, the call fails.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_STATUS = {-1: "sizes or options the kernel does not take", -2: "unsupported element type",
           -3: "pointer or row stride not aligned as the kernel needs"}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = load_library()
        L.cretif_uniform01.restype = ctypes.c_float
        L.cretif_uniform01.argtypes = [ctypes.c_ulonglong, ctypes.c_longlong, ctypes.c_int]
        _lib = L
    return _lib


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (graph replays are not counted)."""
    return _launches


_VARIANTS = ("fused_registers", "fused_row_groups", "fused_cluster2", "fused_cluster4", "stream",
             "stream_row_groups", "decode_cluster", "decode_split", "prefill_attn", "tc64",
             "tc128", "tc256", "tc_several_tiles", "tc192", "prefill_attn_pair",
             "prefill_attn_split", "tc_bulk_add", "tc_pair")


def variant_counts() -> dict:
    """How often each variant of the kernels has been launched so far (the order is that of
    ``cretif::Variant``); tests take differences to know which path a step took.  Launches
    replayed from a CUDA graph are not counted."""
    L = lib()
    return {name: int(L.cretif_variant_count(i)) for i, name in enumerate(_VARIANTS)}


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: {_STATUS.get(code, f'status {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"tensors of dtype {t.dtype} have no kernel") from None


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device as a pointer (the raw getter is an order
    of magnitude cheaper than building a torch.cuda.Stream object for every launch)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    try:
        if t.is_cuda and (dtype is None or t.dtype == dtype) and (dim is None or t.dim() == dim):
            return
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    raise KernelError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride (in elements) of a 2-d tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-d with dense rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0)


# ------------------------------------------------------------------ elementwise
def embed_rows(table, ids, out, fault, positions=None, tok_pos=None) -> None:
    """``positions`` [P, H] (same type as ``table``) with ``tok_pos``: a learned vector per
    position is added to each token's row."""
    _need(table, "table", dim=2); _need(ids, "ids", torch.int32, 1)
    _need(out, "out", torch.float32, 2); _need(fault, "fault", torch.int32)
    T, (V, H) = ids.numel(), table.shape
    if tuple(out.shape) != (T, H) or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError(f"embed_rows: out must be a contiguous [{T}, {H}] tensor")
    P = 0
    if positions is not None:
        _need(positions, "positions", table.dtype, 2); _need(tok_pos, "tok_pos", torch.int32, 1)
        P = positions.shape[0]
        if positions.shape[1] != H or not positions.is_contiguous() or tok_pos.numel() != T:
            raise KernelError(f"embed_rows: positions must be a contiguous [P, {H}] table with "
                              "a position per token")
    _check(lib().cretif_embed_rows(_p(table), _dt(table), _p(ids), _p(out), T, H, V, _p(fault),
                                   _p(positions), _p(tok_pos), P, _stream()), "embed_rows")


def add_rmsnorm(h, delta, weight, out, eps: float, rows=None, write_h: bool = True) -> None:
    _need(h, "h", torch.float32, 2); _need(weight, "weight", torch.float32, 1)
    _need(out, "out", dim=2)
    H = h.shape[1]
    if not h.is_contiguous() or not out.is_contiguous() or weight.numel() != H:
        raise KernelError("add_rmsnorm: h and out must be contiguous and weight have H elements")
    if delta is not None:
        _need(delta, "delta", dim=2)
        if tuple(delta.shape) != tuple(h.shape) or not delta.is_contiguous():
            raise KernelError("add_rmsnorm: delta must match h")
    R = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.numel() != R:
            raise KernelError("add_rmsnorm: one source row per output row")
        write_h = False
    elif R != h.shape[0]:
        raise KernelError("add_rmsnorm: out must have as many rows as h")
    if out.shape[1] != H:
        raise KernelError("add_rmsnorm: out has another width than h")
    _check(lib().cretif_add_rmsnorm(_p(h), _p(delta), _dt(delta) if delta is not None else 0,
                                    _p(weight), _p(out), _dt(out), _p(rows), R, H,
                                    ctypes.c_float(eps), int(write_h), _stream()), "add_rmsnorm")


def silu_mul(gu, act, block: int = 0) -> None:
    """act = silu(gate) * up.  ``block`` = 0: gu rows are [gate | up]; ``block`` = b: groups of b
    gate columns each followed by their b up columns."""
    _need(gu, "gu", dim=2); _need(act, "act", gu.dtype, 2)
    T, I = act.shape
    if tuple(gu.shape) != (T, 2 * I) or not gu.is_contiguous() or not act.is_contiguous():
        raise KernelError(f"silu_mul: gu must be contiguous [{T}, {2 * I}]")
    _check(lib().cretif_silu_mul(_p(gu), _p(act), _dt(gu), T, I, block, _stream()), "silu_mul")


def rope_kv_append(qkv, cos, sin, pairing: int, rot_dim: int, nh: int, nkv: int, hd: int,
                   tok_pos, tok_seq=None, seq_slot=None, table=None, kc=None, vc=None,
                   block_tokens: int = 64, write_cache: bool = True, fault=None,
                   rotate_k_in_place: bool = False) -> None:
    """Position-encode q (in place) and k of the packed ``[T, (nh + 2 nkv) hd]`` rows by a
    rotation table, and/or store k and v at each token's position in the block cache.
    ``write_cache``: rotated k, and v, go to the cache; ``rotate_k_in_place``: k is rotated in
    the buffer as well (encoding alone).  ``rot_dim`` 0 rotates nothing (storing alone)."""
    _need(qkv, "qkv", dim=2)
    T, ld = qkv.shape[0], _rows(qkv, "qkv")
    if rot_dim:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if (cos.shape[1] != rot_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous()):
            raise KernelError("rope_kv_append: cos/sin must be contiguous [positions, rot_dim/2]")
    else:
        cos = sin = None                       # nothing is rotated: the tables are not read
    _need(tok_pos, "tok_pos", torch.int32, 1)
    if write_cache:
        for t, n in ((tok_seq, "tok_seq"), (seq_slot, "seq_slot")):
            _need(t, n, torch.int32, 1)
        _need(table, "table", torch.int32, 2)
        _need(kc, "k cache", qkv.dtype, 4); _need(vc, "v cache", qkv.dtype, 4)
        if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
                or not vc.is_contiguous() or kc.shape != vc.shape):
            raise KernelError("rope_kv_append: cache must be contiguous "
                              f"[blocks, {nkv}, {block_tokens}, {hd}], got {tuple(kc.shape)}")
    if fault is None:
        fault = fault_word(qkv.device)
    flags = (1 if write_cache else 0) | (2 if rotate_k_in_place else 0)
    _check(lib().cretif_rope_kv_append(
        _p(qkv), ld, _dt(qkv), _p(cos), _p(sin), pairing, rot_dim, nh, nkv, hd, _p(tok_pos),
        _p(tok_seq), _p(seq_slot), _p(table), table.stride(0) if table is not None else 0,
        _p(kc), _p(vc), block_tokens, flags, T, _p(fault), _stream()), "rope_kv_append")


def advance_decode(tok_ids, tok_pos, seq_start, sampled, B: int) -> None:
    _check(lib().cretif_advance_decode(_p(tok_ids), _p(tok_pos), _p(seq_start), _p(sampled), B,
                                       _stream()), "advance_decode")


# ------------------------------------------------------------------ matrix products
def gemm_simt(a, w, c, accumulate: bool = False) -> None:
    """c[M,N] (+)= a[M,K] · w[N,K]ᵀ in 32-bit FMA arithmetic."""
    _need(a, "a", dim=2); _need(w, "w", dim=2); _need(c, "c", dim=2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(c.shape) != (M, N):
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(c.shape)}")
    _check(lib().cretif_gemm_simt(_p(a), _dt(a), _p(w), _dt(w), _p(c), _dt(c), M, N, K,
                                  _rows(a, "a"), _rows(w, "w"), _rows(c, "c"), int(accumulate),
                                  _stream()), "gemm_simt")


_batched_simt_only = False


def batched_products_simt_only(on: bool) -> None:
    """(For tests that run both.)  Keep bfloat16 batched products off the tensor cores."""
    global _batched_simt_only
    _batched_simt_only = bool(on)


def gemm_batched(a, w, c) -> None:
    """c[:, z, :] = a[:, z, :] · w[z]ᵀ for every z: ``a`` [M, Z, K], ``w`` [Z, N, K], ``c``
    [M, Z, N] (a matrix per head applied to that head's slice of every row): bfloat16 on the
    tensor cores, float32 by 32-bit FMA."""
    _need(a, "a", dim=3); _need(w, "w", dim=3); _need(c, "c", dim=3)
    M, Z, K = a.shape
    N = w.shape[1]
    if tuple(w.shape) != (Z, N, K) or tuple(c.shape) != (M, Z, N):
        raise KernelError(f"gemm_batched: shapes {tuple(a.shape)} x {tuple(w.shape)} -> "
                          f"{tuple(c.shape)}")
    if a.stride(2) != 1 or c.stride(2) != 1 or not w.is_contiguous():
        raise KernelError("gemm_batched: rows must be dense and w contiguous")
    if a.dtype == w.dtype == c.dtype == torch.bfloat16 and not _batched_simt_only:
        _check(lib().cretif_gemm_heads(
            _p(a), _p(w), _p(c), M, N, K, a.stride(0), c.stride(0), Z,
            ctypes.c_longlong(a.stride(1)), ctypes.c_longlong(c.stride(1)), _stream()),
            "gemm_heads")
        return
    _check(lib().cretif_gemm_simt_batched(
        _p(a), _dt(a), _p(w), _dt(w), _p(c), _dt(c), M, N, K, a.stride(0), K, c.stride(0), Z,
        ctypes.c_longlong(a.stride(1)), ctypes.c_longlong(N * K), ctypes.c_longlong(c.stride(1)),
        _stream()), "gemm_simt_batched")


# ------------------------------------------------------------------ norms beside the sublayers
def rmsnorm_add(h, y, weight, eps: float, x_out=None) -> None:
    """h += y * weight * rsqrt(mean(y²) + eps), row by row, in 32-bit.  ``x_out`` (bfloat16,
    optional) receives the new rows of ``h`` for the sublayer that reads the stream next."""
    _need(h, "h", torch.float32, 2); _need(y, "y", dim=2); _need(weight, "weight", torch.float32, 1)
    R, H = h.shape
    if tuple(y.shape) != (R, H) or not h.is_contiguous() or weight.numel() != H:
        raise KernelError("rmsnorm_add: y must match h and weight have H elements")
    if x_out is not None:
        _need(x_out, "x_out", torch.bfloat16, 2)
        if tuple(x_out.shape) != (R, H) or not x_out.is_contiguous():
            raise KernelError("rmsnorm_add: x_out must be a contiguous copy of h's shape")
    _check(lib().cretif_rmsnorm_add(_p(h), _p(y), _dt(y), _rows(y, "y"), _p(weight), R, H,
                                    ctypes.c_float(eps), _p(x_out), _stream()), "rmsnorm_add")


def convert_rows(h, out) -> None:
    """out = h in out's element type."""
    _need(h, "h", torch.float32); _need(out, "out")
    if h.shape != out.shape or not h.is_contiguous() or not out.is_contiguous():
        raise KernelError("convert_rows: out must match h, both contiguous")
    _check(lib().cretif_convert_rows(_p(h), _p(out), _dt(out), ctypes.c_longlong(h.numel()),
                                     _stream()), "convert_rows")


def proj_norm_kv_append(rows, q_dim: int, wq, nkv: int, hd: int, wk, eps: float, tok_pos, tok_seq,
                        seq_slot, table, kc, vc, block_tokens: int, write_cache: bool,
                        fault) -> None:
    """``rows`` [T, q_dim + nkv·hd + …]: with ``wq`` the first q_dim columns are RMS-normed as
    one vector (times wq) in place; the next nkv·hd columns, normed as one vector (times wk), go
    to the key cache, and as they are to the value cache when ``vc`` is given."""
    _need(rows, "rows", dim=2); _need(wk, "wk", torch.float32, 1)
    if wq is not None:
        _need(wq, "wq", torch.float32, 1)
        if wq.numel() != q_dim:
            raise KernelError("proj_norm_kv_append: wq has one weight per query column")
    if wk.numel() != nkv * hd or rows.shape[1] < q_dim + nkv * hd:
        raise KernelError("proj_norm_kv_append: sizes do not fit")
    _need(kc, "k cache", rows.dtype, 4)
    if tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous():
        raise KernelError("proj_norm_kv_append: cache must be contiguous "
                          f"[blocks, {nkv}, {block_tokens}, {hd}]")
    if vc is not None:
        _need(vc, "v cache", rows.dtype, 4)
        if vc.shape != kc.shape or not vc.is_contiguous():
            raise KernelError("proj_norm_kv_append: the value cache must match the key cache")
    _check(lib().cretif_proj_norm_kv_append(
        _p(rows), _rows(rows, "rows"), _dt(rows), q_dim, _p(wq), nkv, hd, _p(wk),
        ctypes.c_float(eps), _p(tok_pos), _p(tok_seq), _p(seq_slot), _p(table), table.stride(0),
        _p(kc), _p(vc), block_tokens, int(write_cache), rows.shape[0], _p(fault), _stream()),
        "proj_norm_kv_append")


# ------------------------------------------------------------------ gated delta rule
def delta_prepare(proj, prep, conv_w, conv_state, a_log, dt_bias, ctx_pos, ctx_seq, seq_slot,
                  seq_start, H: int, G: int, d: int, e: int, unit_eps: float) -> None:
    """Convolution over time, SiLU, unit-length q/k, beta and decay of every token.  ``proj``
    [T, 2Gd + 2He + 2H] and ``prep`` [T, 2Gd + He + 2H] float32; ``conv_state``
    [slots, …] is the view of the slots' saved inputs ([C, taps-1] each)."""
    _need(proj, "proj", torch.float32, 2); _need(prep, "prep", torch.float32, 2)
    _need(conv_w, "conv_w", torch.float32, 2); _need(conv_state, "conv_state", torch.float32, 2)
    C, taps = conv_w.shape
    if (C != 2 * G * d + H * e or not conv_w.is_contiguous() or conv_state.stride(1) != 1
            or conv_state.shape[1] != C * (taps - 1)):
        raise KernelError("delta_prepare: the convolution's sizes do not fit")
    _check(lib().cretif_delta_prepare(
        _p(proj), _rows(proj, "proj"), _p(prep), _rows(prep, "prep"), _p(conv_w), taps,
        _p(conv_state), ctypes.c_longlong(conv_state.stride(0)), _p(a_log), _p(dt_bias),
        _p(ctx_pos), _p(ctx_seq), _p(seq_slot), _p(seq_start), H, G, d, e,
        ctypes.c_float(unit_eps), proj.shape[0], _stream()), "delta_prepare")


def delta_conv_state(proj, conv_state, taps: int, C: int, cu_seqlens, seq_slot, B: int) -> None:
    """Save every sequence's last taps-1 inputs of the C convolved channels."""
    _need(proj, "proj", torch.float32, 2); _need(conv_state, "conv_state", torch.float32, 2)
    _check(lib().cretif_delta_conv_state(
        _p(proj), _rows(proj, "proj"), _p(conv_state), ctypes.c_longlong(conv_state.stride(0)),
        taps, C, _p(cu_seqlens), _p(seq_slot), B, _stream()), "delta_conv_state")


def delta_recurrence(prep, gate, state, cu_seqlens, seq_slot, B: int, H: int, G: int, d: int,
                     e: int, norm_w, eps: float, out, write_state: bool = True) -> None:
    """The recurrence over the step's tokens of every (sequence, head), from and to ``state``
    (view [slots, H·d·e] float32), then the per-head RMS norm times ``norm_w`` times
    SiLU(``gate``) → ``out`` [T, H·e]."""
    _need(prep, "prep", torch.float32, 2); _need(gate, "gate", torch.float32, 2)
    _need(state, "state", torch.float32, 2); _need(out, "out", dim=2)
    _need(norm_w, "norm_w", torch.float32, 1)
    if state.stride(1) != 1 or state.shape[1] != H * d * e or norm_w.numel() != e:
        raise KernelError("delta_recurrence: the state's sizes do not fit")
    T = prep.shape[0]
    o_raw = torch.empty((T, H * e), dtype=torch.float32, device=prep.device)
    _check(lib().cretif_delta_recurrence(
        _p(prep), _rows(prep, "prep"), _p(gate), _rows(gate, "gate"), _p(state),
        ctypes.c_longlong(state.stride(0)), _p(cu_seqlens), _p(seq_slot), B, H, G, d, e,
        _p(norm_w), ctypes.c_float(eps), _p(o_raw), _p(out), _dt(out), _rows(out, "out"),
        int(write_state), T, _stream()), "delta_recurrence", kernels=2)


# ------------------------------------------------------------------ per-head work, retention
def headnorm_rope_kv_append(proj, bias, wq, wk, eps: float, cos, sin, pairing: int, rot_dim: int,
                            tok_pos, tok_seq, seq_slot, nh: int, nkv: int, hd: int, vd: int,
                            q_out, table=None, kc=None, vc=None, block_tokens: int = 64,
                            write_cache: bool = True, fault=None) -> None:
    """``proj`` rows [q (nh hd) | k (nkv hd) | v (nkv vd) | ...] (float32, or the type of
    ``q_out``): + ``bias``, RMS norm of every q and k head times ``wq`` / ``wk`` (float32 [hd],
    both None for no norm), rotation of each head's first ``rot_dim`` channels by the position;
    q to ``q_out`` [T, nh hd], k and v into the block cache."""
    _need(proj, "proj", dim=2); _need(q_out, "q_out", dim=2)
    T = proj.shape[0]
    if proj.dtype not in (torch.float32, q_out.dtype):
        raise KernelError("headnorm_rope_kv_append: proj is float32 or of q_out's type")
    n_in = (nh + nkv) * hd + nkv * vd
    if q_out.shape[0] != T or q_out.shape[1] < nh * hd or proj.shape[1] < n_in:
        raise KernelError("headnorm_rope_kv_append: proj or q_out too narrow")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.numel() < n_in or not bias.is_contiguous():
            raise KernelError("headnorm_rope_kv_append: the bias has a number per q, k and v "
                              "column")
    if (wq is None) != (wk is None):
        raise KernelError("headnorm_rope_kv_append: norm weights for q and k, or for neither")
    if wq is not None:
        _need(wq, "wq", torch.float32, 1); _need(wk, "wk", torch.float32, 1)
        if wq.numel() != hd or wk.numel() != hd:
            raise KernelError("headnorm_rope_kv_append: a norm weight has head_dim numbers")
    if rot_dim:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError("headnorm_rope_kv_append: cos/sin must be contiguous "
                              "[positions, rot_dim/2]")
    else:
        cos = sin = None
    _need(tok_pos, "tok_pos", torch.int32, 1)
    if write_cache:
        _need(tok_seq, "tok_seq", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
        _need(table, "table", torch.int32, 2)
        _need(kc, "k cache", q_out.dtype, 4); _need(vc, "v cache", q_out.dtype, 4)
        if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
                or tuple(vc.shape[1:]) != (nkv, block_tokens, vd) or not vc.is_contiguous()):
            raise KernelError("headnorm_rope_kv_append: caches must be contiguous [blocks, "
                              f"{nkv}, {block_tokens}, {hd}] and [..., {vd}]")
    if fault is None:
        fault = fault_word(proj.device)
    _check(lib().cretif_headnorm_rope_kv_append(
        _p(proj), _rows(proj, "proj"), _dt(proj), _p(bias), _p(wq), _p(wk), ctypes.c_float(eps),
        _p(cos), _p(sin), pairing, rot_dim, _p(tok_pos), _p(tok_seq), _p(seq_slot), nh, nkv, hd,
        vd, _p(q_out), _rows(q_out, "q_out"), _dt(q_out), _p(table),
        table.stride(0) if table is not None else 0, _p(kc), _p(vc), block_tokens,
        int(write_cache), T, _p(fault), _stream()), "headnorm_rope_kv_append")


def latent_in(proj, q_rank: int, rank: int, rot: int, wq, wc, eps: float, cos, sin, pairing: int,
              tok_pos, tok_seq, seq_slot, cq_out, table=None, kc=None, block_tokens: int = 64,
              write_cache: bool = True, fault=None, rot_dims: Optional[int] = None) -> None:
    """``proj`` rows [cq (q_rank) | c (rank) | kr (rot) | ...] (float32, or the cache's type):
    cq and c to unit RMS times ``wq`` / ``wc`` (float32), kr rotated by the position (its first
    ``rot_dims`` channels, all of them by default; the rest pass); cq to
    ``cq_out`` [T, q_rank] (``q_rank`` 0: no query latent), [c | kr] into the token's row of the
    key cache ``kc`` [blocks, 1, block_tokens, rank + rot]."""
    _need(proj, "proj", dim=2); _need(wc, "wc", torch.float32, 1)
    T = proj.shape[0]
    dt = kc.dtype if kc is not None else cq_out.dtype
    if proj.dtype not in (torch.float32, dt) or proj.shape[1] < q_rank + rank + rot:
        raise KernelError("latent_in: proj is float32 or of the cache's type and holds "
                          "[cq | c | kr]")
    if wc.numel() != rank or not wc.is_contiguous():
        raise KernelError("latent_in: the latent's norm weight has `rank` numbers")
    if q_rank:
        _need(wq, "wq", torch.float32, 1); _need(cq_out, "cq_out", dt, 2)
        if wq.numel() != q_rank or cq_out.shape[0] != T or cq_out.shape[1] < q_rank \
                or not wq.is_contiguous():
            raise KernelError("latent_in: the query latent's weight and output have q_rank columns")
    rdims = rot if rot_dims is None else int(rot_dims)
    if not 0 <= rdims <= rot or rdims % 2:
        raise KernelError("latent_in: rot_dims is even and at most rot")
    if rdims:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rdims // 2 or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError("latent_in: cos/sin must be contiguous [positions, rot_dims/2]")
    else:
        cos = sin = None
    if write_cache:
        _need(table, "table", torch.int32, 2); _need(kc, "k cache", dt, 4)
        if tuple(kc.shape[1:]) != (1, block_tokens, rank + rot) or not kc.is_contiguous():
            raise KernelError(f"latent_in: the cache must be contiguous [blocks, 1, "
                              f"{block_tokens}, {rank + rot}]")
    if fault is None:
        fault = fault_word(proj.device)
    _check(lib().cretif_latent_in(
        _p(proj), _rows(proj, "proj"), _dt(proj), q_rank, rank, rot, rdims, _p(wq), _p(wc),
        ctypes.c_float(eps), _p(cos), _p(sin), pairing, _p(tok_pos), _p(tok_seq), _p(seq_slot),
        _p(cq_out), _rows(cq_out, "cq_out") if q_rank else 0, _DT[dt], _p(table),
        table.stride(0) if table is not None else 0, _p(kc), block_tokens, int(write_cache), T,
        _p(fault), _stream()), "latent_in")


def rope_heads(q, nh: int, d: int, rot: int, cos, sin, pairing: int, tok_pos, out, off: int,
               rot_dims: Optional[int] = None) -> None:
    """``q`` [T, nh·(d + rot)]: the last ``rot`` channels of every head, rotated by the token's
    position (the first ``rot_dims`` of them, all by default; the rest pass), go to ``out[t, h, off : off + rot]`` (``out`` [T, nh, width >= off + rot], of the
    compute type; ``q`` float32 or of that type)."""
    _need(q, "q", dim=2); _need(out, "out", dim=3)
    T = q.shape[0]
    if (q.shape[1] < nh * (d + rot) or out.shape[0] != T or out.shape[1] != nh
            or out.shape[2] < off + rot or out.stride(2) != 1
            or q.dtype not in (torch.float32, out.dtype)):
        raise KernelError("rope_heads: sizes or element types do not fit")
    if rot == 0:
        return
    rdims = rot if rot_dims is None else int(rot_dims)
    if not 0 <= rdims <= rot or rdims % 2:
        raise KernelError("rope_heads: rot_dims is even and at most rot")
    if rdims:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rdims // 2 or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError("rope_heads: cos/sin must be contiguous [positions, rot_dims/2]")
    else:
        cos = sin = None
    _check(lib().cretif_rope_heads(
        _p(q), _rows(q, "q"), _dt(q), nh, d, rot, rdims, _p(cos), _p(sin), pairing, _p(tok_pos), _p(out),
        out.stride(0), out.stride(1), off, _dt(out), T, _stream()), "rope_heads")


def rmsnorm_rows(x, weight, eps: float) -> None:
    """``x <- x / sqrt(mean(x²) + eps) * weight`` in place on float32 rows."""
    _need(x, "x", torch.float32, 2); _need(weight, "weight", torch.float32, 1)
    if weight.numel() != x.shape[1] or not weight.is_contiguous():
        raise KernelError("rmsnorm_rows: a weight per column")
    _check(lib().cretif_rmsnorm_rows(_p(x), _rows(x, "x"), _p(weight), x.shape[0], x.shape[1],
                                     ctypes.c_float(eps), _stream()), "rmsnorm_rows")


def gate_heads(o, g, nh: int, vd: int) -> None:
    """``o[t, h, :] *= sigmoid(g[t, h])``; ``g`` float32 [T, >= nh] (columns of a projection)."""
    _need(o, "o", dim=2); _need(g, "g", torch.float32, 2)
    if o.shape[1] < nh * vd or g.shape[1] < nh or g.shape[0] != o.shape[0]:
        raise KernelError("gate_heads: o holds [tokens, heads*value_dim], g [tokens, heads]")
    _check(lib().cretif_gate_heads(_p(o), _rows(o, "o"), _dt(o), _p(g), _rows(g, "g"), nh, vd,
                                   o.shape[0], _stream()), "gate_heads")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "gelu": 3}


def activation(x, out, kind: str) -> None:
    """``out = act(x)`` element by element: ``relu2`` (the square of relu), ``gelu_tanh``,
    ``silu``, ``gelu`` (the exact form, with the error function); ``x`` float32 or of ``out``'s type."""
    _need(x, "x", dim=2); _need(out, "out", dim=2)
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: {kind!r} is none of {sorted(ACTIVATIONS)}")
    if x.shape != out.shape or x.dtype not in (torch.float32, out.dtype):
        raise KernelError("activation: out has x's shape, x is float32 or of out's type")
    _check(lib().cretif_activation(_p(x), _rows(x, "x"), _dt(x), _p(out), _rows(out, "out"),
                                   _dt(out), x.shape[0], x.shape[1], ACTIVATIONS[kind],
                                   _stream()), "activation")


def softcap(z, cap: float) -> None:
    """``z <- cap * tanh(z / cap)`` in place (float32, contiguous)."""
    _need(z, "z", torch.float32)
    if not z.is_contiguous():
        raise KernelError("softcap: z must be contiguous")
    _check(lib().cretif_softcap(_p(z), ctypes.c_longlong(z.numel()), ctypes.c_float(cap),
                                _stream()), "softcap")


def axpy_rows(h, y, alpha: float) -> None:
    """``h += alpha * y`` in 32-bit; ``y`` float32 or bfloat16 of ``h``'s shape."""
    _need(h, "h", torch.float32); _need(y, "y")
    if y.shape != h.shape or not h.is_contiguous() or not y.is_contiguous():
        raise KernelError("axpy_rows: y must match h, both contiguous")
    _check(lib().cretif_axpy_rows(_p(h), _p(y), _dt(y), ctypes.c_float(alpha),
                                  ctypes.c_longlong(h.numel()), _stream()), "axpy_rows")


def retention_prepare(proj, prep, cos, sin, pairing: int, rot_dim: int, tok_pos, H: int, d: int,
                      k_scale: float) -> None:
    """Rotate the q and k heads of ``proj`` [T, >= 2Hd] (float32) by position into ``prep``
    [T, 2Hd]; the rotated k is multiplied by ``k_scale``."""
    _need(proj, "proj", torch.float32, 2); _need(prep, "prep", torch.float32, 2)
    if rot_dim:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError("retention_prepare: cos/sin must be contiguous "
                              "[positions, rot_dim/2]")
    else:
        cos = sin = None
    _need(tok_pos, "tok_pos", torch.int32, 1)
    if prep.shape[0] != proj.shape[0]:
        raise KernelError("retention_prepare: a row of prep per row of proj")
    _check(lib().cretif_retention_prepare(
        _p(proj), _rows(proj, "proj"), _p(prep), _rows(prep, "prep"), _p(cos), _p(sin), pairing,
        rot_dim, _p(tok_pos), H, d, ctypes.c_float(k_scale), proj.shape[0], _stream()),
        "retention_prepare")


def retention_recurrence(prep, v, decay, state, cu_seqlens, seq_slot, B: int, H: int, d: int,
                         e: int, o_raw, write_state: bool = True, form: str = "auto") -> None:
    """``S <- decay_h S + k vᵀ; o = Sᵀ q`` over the step's tokens of every (sequence, head), from
    and to ``state`` (view [slots, H·d·e] float32); ``prep`` [T, 2Hd] holds q and k, ``v``
    [T, >= He] the values (float32), ``o_raw`` [T, He] receives the read-outs.  ``form``:
    ``"token"`` walks the tokens one by one, ``"chunk"`` takes 64 at a time as matrix products
    in two kernels (refused where sizes or addresses rule out 16-byte accesses), ``"auto"`` takes
    chunks where the step brings 16 tokens a sequence or more and they are allowed."""
    _need(prep, "prep", torch.float32, 2); _need(v, "v", torch.float32, 2)
    _need(decay, "decay", torch.float32, 1); _need(state, "state", torch.float32, 2)
    _need(o_raw, "o_raw", torch.float32, 2)
    T = prep.shape[0]
    if (state.stride(1) != 1 or state.shape[1] != H * d * e or decay.numel() != H
            or tuple(o_raw.shape) != (T, H * e) or not o_raw.is_contiguous() or v.shape[0] != T):
        raise KernelError("retention_recurrence: the sizes do not fit")
    _check(lib().cretif_retention_recurrence(
        _p(prep), _rows(prep, "prep"), _p(v), _rows(v, "v"), _p(decay), _p(state),
        ctypes.c_longlong(state.stride(0)), _p(cu_seqlens), _p(seq_slot), B, H, d, e, _p(o_raw),
        int(write_state), T, {"auto": 0, "token": 1, "chunk": 2}[form], _stream()),
        "retention_recurrence")


def heads_out_norm(o_raw, gate, norm_w, eps: float, out, H: int, e: int,
                   per_head_weight: bool = False, gate_sigmoid: bool = False) -> None:
    """``out = o_raw / rms(o_raw) [* norm_w] * gate(gate)`` per (token, head) over ``e``
    channels; ``norm_w`` None, [e] or [H·e]; the gate is SiLU or the logistic function."""
    _need(o_raw, "o_raw", torch.float32, 2); _need(gate, "gate", torch.float32, 2)
    _need(out, "out", dim=2)
    T = o_raw.shape[0]
    if (tuple(o_raw.shape) != (T, H * e) or not o_raw.is_contiguous() or gate.shape[0] != T
            or out.shape[0] != T or out.shape[1] < H * e):
        raise KernelError("heads_out_norm: the sizes do not fit")
    if norm_w is not None:
        _need(norm_w, "norm_w", torch.float32, 1)
        if norm_w.numel() != (H * e if per_head_weight else e):
            raise KernelError("heads_out_norm: the weight has e or H·e numbers")
    _check(lib().cretif_heads_out_norm(
        _p(o_raw), _p(gate), _rows(gate, "gate"), _p(norm_w), int(per_head_weight),
        int(gate_sigmoid), ctypes.c_float(eps), _p(out), _dt(out), _rows(out, "out"), H, e, T,
        _stream()), "heads_out_norm")


# ------------------------------------------------------------------ Dynamic Tanh, token shift
def dyt_rows(h, delta, weight, bias, alpha, out, gain=None, rows=None, write_h: bool = True) -> None:
    """out[r] = (tanh(alpha v) w + b) gain with v = h[src] (+ delta[src]); ``alpha`` is a
    one-element float32 tensor on the device."""
    _need(h, "h", torch.float32, 2); _need(out, "out", dim=2)
    H = h.shape[1]
    for name, t in (("weight", weight), ("bias", bias), ("gain", gain)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != H or not t.is_contiguous():
                raise KernelError(f"dyt_rows: {name} must have {H} elements")
    _need(alpha, "alpha", torch.float32)
    if not h.is_contiguous() or not out.is_contiguous() or alpha.numel() != 1:
        raise KernelError("dyt_rows: h and out must be contiguous and alpha one number")
    if delta is not None:
        _need(delta, "delta", dim=2)
        if delta.shape != h.shape or not delta.is_contiguous():
            raise KernelError("dyt_rows: delta must match h")
    R = h.shape[0] if rows is None else rows.numel()
    if tuple(out.shape) != (R, H):
        raise KernelError(f"dyt_rows: out must be [{R}, {H}]")
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    _check(lib().cretif_dyt_rows(
        _p(h), _p(delta), 0 if delta is None else _dt(delta), _p(weight), _p(bias), _p(alpha),
        _p(gain), _p(out), _dt(out), _p(rows), R, H,
        int(write_h and rows is None and delta is not None), _stream()), "dyt_rows")


def dyt_add(h, y, weight, bias, alpha, gain=None) -> None:
    """h += (tanh(alpha y) w + b) gain, element by element, in 32-bit."""
    _need(h, "h", torch.float32, 2); _need(y, "y", dim=2)
    R, H = h.shape
    if tuple(y.shape) != (R, H) or not h.is_contiguous() or weight.numel() != H \
            or bias.numel() != H or (gain is not None and gain.numel() != H) or alpha.numel() != 1:
        raise KernelError("dyt_add: y must match h and the weights have H elements")
    for t in (weight, bias, alpha) + ((gain,) if gain is not None else ()):
        _need(t, "weight", torch.float32)
    _check(lib().cretif_dyt_add(_p(h), _p(y), _dt(y), _rows(y, "y"), _p(weight), _p(bias),
                                _p(alpha), _p(gain), R, H, _stream()), "dyt_add")


def shift_rows(h, shift, state, tok_seq, seq_slot, cu_seqlens, out, weight=None, bias=None,
               alpha=None) -> None:
    """out[t] = n[t] + (n[t-1] - n[t]) * shift, n = dyt(h) when weight/bias/alpha are given, else
    n = h.  A sequence's first token of the step reads ``state[slot]`` (float32 [slots, H]) and
    leaves the step's last row there."""
    _need(h, "h", torch.float32, 2); _need(shift, "shift", torch.float32, 1)
    _need(state, "state", torch.float32, 2); _need(out, "out", dim=2)
    T, H = h.shape
    if (not h.is_contiguous() or not out.is_contiguous() or tuple(out.shape) != (T, H)
            or shift.numel() != H or state.shape[1] != H or state.stride(1) != 1):
        raise KernelError("shift_rows: sizes do not fit")
    if weight is not None:
        for t in (weight, bias, alpha):
            _need(t, "norm weight", torch.float32)
        if weight.numel() != H or bias.numel() != H or alpha.numel() != 1:
            raise KernelError("shift_rows: the norm's weights have H elements")
    _check(lib().cretif_shift_rows(
        _p(h), _p(weight), _p(bias), _p(alpha), _p(shift), _p(state),
        ctypes.c_longlong(state.stride(0)), _p(tok_seq), _p(seq_slot), _p(cu_seqlens), _p(out),
        _dt(out), T, H, _stream()), "shift_rows")


# ------------------------------------------------------------------ convolved attention inputs
def conv_headnorm_kv_append(proj, conv_w, conv_state, tok_pos, tok_seq, seq_slot, seq_start,
                            nh: int, nkv: int, hd: int, vd: int, eps: float, gain_coef: float,
                            gain_every: int, q_out, table=None, kc=None, vc=None,
                            block_tokens: int = 0, write_cache: bool = True, fault=None) -> None:
    """``proj`` float32 [T, nh·hd + nkv·(hd + vd)] -> convolution over time, unit RMS per q/k
    head, the query's gain by position; q into ``q_out``, k and v into the block cache.  ``nkv``
    0: queries only.  ``conv_state`` [slots, C·(taps-1)] holds every slot's last inputs."""
    _need(proj, "proj", torch.float32, 2); _need(conv_w, "conv_w", torch.float32, 2)
    _need(q_out, "q_out", dim=2)
    C, taps = conv_w.shape
    if C != nh * hd + nkv * (hd + vd) or not conv_w.is_contiguous() or proj.shape[1] < C:
        raise KernelError("conv_headnorm_kv_append: the convolution's sizes do not fit")
    if taps > 1:
        _need(conv_state, "conv_state", torch.float32, 2)
        if conv_state.stride(1) != 1 or conv_state.shape[1] != C * (taps - 1):
            raise KernelError("conv_headnorm_kv_append: conv_state must be [slots, C (taps-1)]")
    if q_out.shape[0] != proj.shape[0] or q_out.shape[1] < nh * hd:
        raise KernelError("conv_headnorm_kv_append: q_out must be [tokens, heads*head_dim]")
    if nkv > 0:
        _need(kc, "k cache", q_out.dtype, 4); _need(vc, "v cache", q_out.dtype, 4)
        if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
                or tuple(vc.shape[1:]) != (nkv, block_tokens, vd) or not vc.is_contiguous()):
            raise KernelError("conv_headnorm_kv_append: caches must be contiguous "
                              "[blocks, kv_heads, block, head_dim / value_dim]")
    _check(lib().cretif_conv_headnorm_kv_append(
        _p(proj), _rows(proj, "proj"), _p(conv_w), taps, _p(conv_state if taps > 1 else None),
        ctypes.c_longlong(conv_state.stride(0) if taps > 1 else 0), _p(tok_pos), _p(tok_seq),
        _p(seq_slot), _p(seq_start), nh, nkv, hd, vd, ctypes.c_float(eps),
        ctypes.c_float(gain_coef), int(gain_every), _p(q_out), _rows(q_out, "q_out"), _dt(q_out),
        _p(table), 0 if table is None else table.stride(0), _p(kc), _p(vc), block_tokens,
        int(write_cache), proj.shape[0], _p(fault), _stream()), "conv_headnorm_kv_append")


# ------------------------------------------------------------------ generalized delta rule
def tanh_cols(rows, out) -> None:
    """out = tanh(rows) for a strided float32 [T, R] view, in out's element type."""
    _need(rows, "rows", torch.float32, 2); _need(out, "out", dim=2)
    if out.shape != rows.shape or not out.is_contiguous():
        raise KernelError("tanh_cols: out must be a contiguous tensor of rows' shape")
    _check(lib().cretif_tanh_cols(_p(rows), _rows(rows, "rows"), _p(out), _dt(out), rows.shape[1],
                                  rows.shape[0], _stream()), "tanh_cols")


def general_delta_prepare(proj, prep, a_bias, z, w0, H: int, d: int, e: int, unit_eps: float,
                          decay_scale: float) -> None:
    """``proj`` float32 [T, 3Hd + 2He + ...] = [r | k | v | gate | a | ...]; ``z`` [T, Hd] the
    decay's expanded low-rank product; ``prep`` [T, 3Hd] = [unit key | removal along it |
    decay], see delta_rule.cu."""
    _need(proj, "proj", torch.float32, 2); _need(prep, "prep", torch.float32, 2)
    _need(z, "z", torch.float32, 2); _need(w0, "w0", torch.float32, 1)
    _need(a_bias, "a_bias", torch.float32, 1)
    if (z.shape[1] < H * d or z.shape[0] != proj.shape[0] or w0.numel() != H * d
            or a_bias.numel() != H * d or proj.shape[1] < 3 * H * d + 2 * H * e
            or prep.shape[1] < 3 * H * d or prep.shape[0] != proj.shape[0]):
        raise KernelError("general_delta_prepare: sizes do not fit")
    _check(lib().cretif_general_delta_prepare(
        _p(proj), _rows(proj, "proj"), _p(prep), _rows(prep, "prep"), _p(a_bias), _p(z),
        _rows(z, "z"), _p(w0), H, d, e, ctypes.c_float(unit_eps), ctypes.c_float(decay_scale),
        proj.shape[0], _stream()), "general_delta_prepare")


def general_delta_recurrence(proj, prep, gate, state, cu_seqlens, seq_slot, B: int, H: int, d: int,
                             e: int, norm_w, eps: float, out, per_head_weight: bool = True,
                             gate_sigmoid: bool = True, write_state: bool = True) -> None:
    """The generalized delta rule over the step's tokens of every (sequence, head), from and to
    ``state`` (view [slots, H·d·e] float32), then the per-head RMS norm times ``norm_w`` times
    the gate -> ``out`` [T, H·e]."""
    _need(proj, "proj", torch.float32, 2); _need(prep, "prep", torch.float32, 2)
    _need(gate, "gate", torch.float32, 2); _need(state, "state", torch.float32, 2)
    _need(out, "out", dim=2); _need(norm_w, "norm_w", torch.float32, 1)
    T = proj.shape[0]
    if (state.stride(1) != 1 or state.shape[1] < H * d * e or out.shape[0] != T
            or out.shape[1] < H * e or norm_w.numel() != (H * e if per_head_weight else e)):
        raise KernelError("general_delta_recurrence: sizes do not fit")
    o_raw = torch.empty((T, H * e), dtype=torch.float32, device=proj.device)
    _check(lib().cretif_general_delta_recurrence(
        _p(proj), _rows(proj, "proj"), _p(prep), _rows(prep, "prep"), _p(gate),
        _rows(gate, "gate"), _p(state), ctypes.c_longlong(state.stride(0)), _p(cu_seqlens),
        _p(seq_slot), B, H, d, e, _p(norm_w), int(per_head_weight), int(gate_sigmoid),
        ctypes.c_float(eps), _p(o_raw), _p(out), _dt(out), _rows(out, "out"), int(write_state), T,
        _stream()), "general_delta_recurrence", kernels=2)


# ------------------------------------------------------------------ routed experts
MOE_TILE = 64
_moe_simt_only = False


def moe_simt_only(on: bool) -> None:
    """Run the experts' products on the CUDA cores whatever the element type (the yardstick)."""
    global _moe_simt_only
    _moe_simt_only = bool(on)


def moe_max_tiles(pairs: int, experts: int) -> int:
    return -(-pairs // MOE_TILE) + experts


def _route_rule(E: int, top: int, groups: int, keep: int) -> None:
    if groups > 1 and (E % groups or not 1 <= keep <= groups or keep * (E // groups) < top):
        raise KernelError(f"routing: {E} experts do not form {groups} equal groups of which "
                          f"{keep} hold {top} experts")


def moe_route(x, router_w, top: int, ids, wts, renorm: bool = False, groups: int = 0,
              keep: int = 0, sum_eps: float = 0.0) -> None:
    """ids/wts [T, top]: the ``top`` experts with the largest sigmoid(router_w · x) per token.
    ``groups`` > 1: the experts form that many equal groups of neighbours, a group's score is
    the sum of its two largest scores, and only experts of the ``keep`` best groups can be
    chosen.  ``renorm``: the weights are divided by (their sum + ``sum_eps``)."""
    _need(x, "x", dim=2); _need(router_w, "router_w", torch.float32, 2)
    _need(ids, "ids", torch.int32, 2); _need(wts, "wts", torch.float32, 2)
    T, H = x.shape
    E = router_w.shape[0]
    if (router_w.shape[1] != H or not router_w.is_contiguous() or tuple(ids.shape) != (T, top)
            or tuple(wts.shape) != (T, top) or not ids.is_contiguous() or not wts.is_contiguous()):
        raise KernelError("moe_route: sizes do not fit")
    if not 0 < top <= E or E > 256:
        raise KernelError(f"moe_route: {top} of {E} experts (at most 256) cannot be chosen")
    _route_rule(E, top, groups, keep)
    _check(lib().cretif_moe_route(_p(x), _dt(x), _rows(x, "x"), _p(router_w), E, H, top,
                                  int(renorm), int(groups), int(keep), ctypes.c_float(sum_eps),
                                  _p(ids), _p(wts), T, _stream()), "moe_route")


def moe_topk(logits, top: int, ids, wts, renorm: bool = False, groups: int = 0, keep: int = 0,
             sum_eps: float = 0.0) -> None:
    """``moe_route``'s choice from router logits [T, E] (float32) that a matrix product left."""
    _need(logits, "logits", torch.float32, 2); _need(ids, "ids", torch.int32, 2)
    _need(wts, "wts", torch.float32, 2)
    T, E = logits.shape
    if (tuple(ids.shape) != (T, top) or tuple(wts.shape) != (T, top) or not ids.is_contiguous()
            or not wts.is_contiguous() or not 0 < top <= E or E > 256):
        raise KernelError("moe_topk: sizes do not fit")
    _route_rule(E, top, groups, keep)
    _check(lib().cretif_moe_topk(_p(logits), _rows(logits, "logits"), E, top, int(renorm),
                                 int(groups), int(keep), ctypes.c_float(sum_eps), _p(ids),
                                 _p(wts), T, _stream()), "moe_topk")


def moe_group(ids, experts: int, offsets, place, order, tile_expert, tile_row0) -> None:
    """Sort the (token, choice) pairs by expert: ``offsets`` [E + 1], ``place`` [P] (a pair's
    row in the sorted list), ``order`` [P] (its inverse) and the list of 64-row tiles."""
    for name, t in (("ids", ids), ("offsets", offsets), ("place", place), ("order", order),
                    ("tile_expert", tile_expert), ("tile_row0", tile_row0)):
        _need(t, name, torch.int32)
        if not t.is_contiguous():
            raise KernelError(f"moe_group: {name} must be contiguous")
    P = ids.numel()
    if (offsets.numel() != experts + 1 or place.numel() != P or order.numel() != P
            or tile_expert.numel() != tile_row0.numel()
            or tile_expert.numel() < moe_max_tiles(P, experts)):
        raise KernelError("moe_group: sizes do not fit")
    _check(lib().cretif_moe_group(_p(ids), P, experts, _p(offsets), _p(place), _p(order),
                                  _p(tile_expert), _p(tile_row0), tile_expert.numel(), _stream()),
           "moe_group")


def moe_act_mode(kind: str) -> int:
    """The ``mode`` of ``moe_gemm`` / ``moe_gemv`` for the first product of experts without a
    gate whose activation is ``kind`` (a key of ACTIVATIONS)."""
    return 2 + ACTIVATIONS[kind]


def moe_gemm(a, w, c, top: int, mode: int, scale_at: int, wts, order, offsets, tile_expert,
             tile_row0) -> None:
    """Grouped product over the sorted rows.  mode 0: ``a`` [tokens, K], ``w`` [E, 2N, K]
    (gate rows then up rows), ``c`` [P, N] = silu(s g)(s u) (scale_at 1) or silu(g) u; mode 1:
    ``a`` [P, K] sorted rows, ``w`` [E, N, K], ``c`` [P, N] float32 (scale_at 2: times s);
    mode ``moe_act_mode(kind)``: experts without a gate, ``a`` as in mode 0, ``w`` [E, N, K],
    ``c`` = act(s · product)."""
    _need(a, "a", dim=2); _need(w, "w", a.dtype, 3); _need(c, "c", dim=2)
    K = a.shape[1]
    N = c.shape[1]
    if (w.shape[2] != K or w.shape[1] != (2 * N if mode == 0 else N) or not w.is_contiguous()
            or c.dtype != (a.dtype if mode != 1 else torch.float32) or c.shape[0] != order.numel()):
        raise KernelError("moe_gemm: sizes or element types do not fit")
    use_mma = int(a.dtype == torch.bfloat16 and not _moe_simt_only)
    _check(lib().cretif_moe_gemm(
        _p(a), _dt(a), _rows(a, "a"), _p(w), _dt(w), _p(c), _rows(c, "c"), N, K, top, mode,
        scale_at, _p(wts), _p(order), _p(offsets), _p(tile_expert), _p(tile_row0),
        tile_expert.numel(), use_mma, _stream()), "moe_gemm")


def moe_gemv(a, w, c, top: int, mode: int, scale_at: int, ids, wts) -> None:
    """``moe_gemm`` for a handful of pairs, in the pairs' own order (nothing is sorted): a CTA
    per pair and 16 output columns streams the expert's rows once."""
    _need(a, "a", dim=2); _need(w, "w", a.dtype, 3); _need(c, "c", dim=2)
    _need(ids, "ids", torch.int32); _need(wts, "wts", torch.float32)
    K, N, P = a.shape[1], c.shape[1], ids.numel()
    if (w.shape[2] != K or w.shape[1] != (2 * N if mode == 0 else N) or not w.is_contiguous()
            or c.dtype != (a.dtype if mode != 1 else torch.float32) or c.shape[0] != P
            or wts.numel() != P or not ids.is_contiguous() or not wts.is_contiguous()):
        raise KernelError("moe_gemv: sizes or element types do not fit")
    _check(lib().cretif_moe_gemv(
        _p(a), _dt(a), _rows(a, "a"), _p(w), _dt(w), _p(c), _rows(c, "c"), N, K, top, mode,
        scale_at, _p(ids), _p(wts), P, _stream()), "moe_gemv")


MOE_TC_TILE = 128


def moe_tc_tiles(pairs: int, experts: int) -> int:
    """Row tiles of the padded order: every expert may leave one tile partly empty."""
    return -(-pairs // MOE_TC_TILE) + experts


def moe_group_padded(ids, experts: int, place, tile_expert, used) -> None:
    """The order for the tensor-core grouped products: every expert's rows start at a multiple
    of 128; ``place`` [P] is a pair's row, ``tile_expert`` [tiles] a tile's expert (-1: unused),
    ``used`` [1] the number of tiles in use."""
    for name, t in (("ids", ids), ("place", place), ("tile_expert", tile_expert), ("used", used)):
        _need(t, name, torch.int32)
        if not t.is_contiguous():
            raise KernelError(f"moe_group_padded: {name} must be contiguous")
    P = ids.numel()
    if place.numel() != P or tile_expert.numel() < moe_tc_tiles(P, experts) or used.numel() != 1:
        raise KernelError("moe_group_padded: sizes do not fit")
    _check(lib().cretif_moe_group_padded(_p(ids), P, experts, MOE_TC_TILE, _p(place),
                                         _p(tile_expert), tile_expert.numel(), _p(used),
                                         _stream()), "moe_group_padded")


def moe_gather_rows(x, xs, place, wts, top: int) -> None:
    """xs[place[p]] = x[p // top] * wts[p] (``wts`` None: as it is), bfloat16."""
    _need(x, "x", torch.bfloat16, 2); _need(xs, "xs", torch.bfloat16, 2)
    _need(place, "place", torch.int32)
    if xs.shape[1] != x.shape[1] or place.numel() != x.shape[0] * top:
        raise KernelError("moe_gather_rows: sizes do not fit")
    _check(lib().cretif_moe_gather_rows(_p(x), _rows(x, "x"), _p(xs), _rows(xs, "xs"), _p(place),
                                        _p(wts), top, x.shape[1], place.numel(), _stream()),
           "moe_gather_rows")


def moe_tc_supported(x, w_gu, w_down, gated: bool = True) -> bool:
    """Whether the grouped tensor-core products take these operands (bfloat16, widths that are
    multiples of 8, an expert width that is a multiple of 64)."""
    K, F = x.shape[1], w_down.shape[2]
    return (x.dtype == torch.bfloat16 and w_gu.dtype == torch.bfloat16 and K % 8 == 0
            and F % (64 if gated else 8) == 0 and not _moe_simt_only)


def gemm_tc_silu_grouped(xs, w_gu, act, tile_expert, used) -> None:
    """act = silu(xs Wg[e]ᵀ) ⊙ (xs Wu[e]ᵀ) tile by tile; ``w_gu`` [E, 2F, K] with gate and up
    rows interleaved in blocks of 64 inside each expert."""
    _need(xs, "xs", torch.bfloat16, 2); _need(w_gu, "w_gu", torch.bfloat16, 3)
    _need(act, "act", torch.bfloat16, 2)
    M, K = xs.shape
    E, F = w_gu.shape[0], w_gu.shape[1] // 2
    if (M % MOE_TC_TILE or tuple(act.shape) != (M, F) or w_gu.shape[2] != K
            or not w_gu.is_contiguous() or not act.is_contiguous()
            or tile_expert.numel() < M // MOE_TC_TILE):
        raise KernelError("gemm_tc_silu_grouped: sizes do not fit")
    _check(lib().cretif_gemm_tc_silu_grouped(
        _p(xs), _p(w_gu), _p(act), M, F, K, _rows(xs, "xs"), K, E, _p(tile_expert), _p(used),
        _p(fault_word(xs.device)), _stream()), "gemm_tc_silu_grouped")


def gemm_tc_act_grouped(a, w, c, tile_expert, used, kind: str) -> None:
    """c (bfloat16) = act(a W[e]ᵀ) tile by tile; ``w`` [E, N, K], ``kind`` a key of ACTIVATIONS."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 3)
    _need(c, "c", torch.bfloat16, 2)
    M, K = a.shape
    E, N = w.shape[0], w.shape[1]
    if (M % MOE_TC_TILE or tuple(c.shape) != (M, N) or w.shape[2] != K or not w.is_contiguous()
            or tile_expert.numel() < M // MOE_TC_TILE):
        raise KernelError("gemm_tc_act_grouped: sizes do not fit")
    _check(lib().cretif_gemm_tc_act_grouped(
        _p(a), _p(w), _p(c), M, N, K, _rows(a, "a"), K, _rows(c, "c"), E, _p(tile_expert),
        _p(used), 1 + ACTIVATIONS[kind], _p(fault_word(a.device)), _stream()),
        "gemm_tc_act_grouped")


def gemm_tc_grouped(a, w, c, tile_expert, used) -> None:
    """c (float32) = a W[e]ᵀ tile by tile; ``w`` [E, N, K]."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 3)
    _need(c, "c", torch.float32, 2)
    M, K = a.shape
    E, N = w.shape[0], w.shape[1]
    if (M % MOE_TC_TILE or tuple(c.shape) != (M, N) or w.shape[2] != K or not w.is_contiguous()
            or tile_expert.numel() < M // MOE_TC_TILE):
        raise KernelError("gemm_tc_grouped: sizes do not fit")
    _check(lib().cretif_gemm_tc_grouped(
        _p(a), _p(w), _p(c), M, N, K, _rows(a, "a"), K, _rows(c, "c"), E, _p(tile_expert),
        _p(used), _p(fault_word(a.device)), _stream()), "gemm_tc_grouped")


def moe_combine(rows, place, top: int, y, wts=None) -> None:
    """y[t] = the sum of the token's ``top`` rows of ``rows`` (float32), in their order, each
    times its weight when ``wts`` is given; ``place`` None: the rows are in the pairs' own
    order."""
    _need(rows, "rows", torch.float32, 2); _need(y, "y", torch.float32, 2)
    if place is not None:
        _need(place, "place", torch.int32)
    T, H = y.shape
    if (rows.shape[1] != H or (place is not None and place.numel() != T * top)
            or rows.shape[0] < T * top or not y.is_contiguous()):
        raise KernelError("moe_combine: sizes do not fit")
    _check(lib().cretif_moe_combine(_p(rows), _rows(rows, "rows"), _p(place), top, _p(wts), _p(y),
                                    T, H, _stream()), "moe_combine")


# ------------------------------------------------------------------ attention
def attn_simt(q, out, kc, vc, table, tok_pos, tok_seq, seq_slot, nh: int, nkv: int, hd: int,
              scale: float, window: int, block_tokens: int, sink=None, vd: int = 0, bias=None,
              bias_edges=None, slope=None) -> None:
    """``window`` > 0: a sliding window of that many keys; < 0: chunks of ``-window`` positions
    counted from 0, a query sees the keys of its own chunk; 0: every earlier key.  ``slope``
    (float32 [heads], optional): the key n positions back has ``slope[h] * n`` taken off its
    scaled score.  ``sink`` (float32 [heads], optional): exp(sink_h) joins head h's softmax denominator
    without a key or a value.  ``vd``: size of a value head when it is not ``hd``.  ``bias``
    (float32 [rows, heads]) with ``bias_edges`` (int32 [rows], ascending from 0): the key n
    positions back adds ``bias[r, h]`` to its scaled score, r the last row with edge <= n."""
    _need(q, "q", dim=2); _need(out, "out", q.dtype, 2)
    _need(kc, "k cache", q.dtype, 4); _need(vc, "v cache", q.dtype, 4)
    T = q.shape[0]
    vd = vd or hd
    if out.shape[0] != T or out.shape[1] < nh * vd or q.shape[1] < nh * hd:
        raise KernelError("attention: q must hold [tokens, heads*head_dim], out "
                          "[tokens, heads*value_dim]")
    if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
            or tuple(vc.shape[1:]) != (nkv, block_tokens, vd) or not vc.is_contiguous()):
        raise KernelError("attention: caches must be contiguous [blocks, kv_heads, block, "
                          "head_dim] and [..., value_dim]")
    if hd <= 0 or hd > 512 or vd > 512:
        raise KernelError(f"attention: head sizes {hd}, {vd} are not in [1, 512]")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.numel() != nh or not sink.is_contiguous():
            raise KernelError("attention: the sink has one number per query head")
    rows = 0
    if bias is not None:
        _need(bias, "bias", torch.float32, 2); _need(bias_edges, "bias_edges", torch.int32, 1)
        rows = bias.shape[0]
        if (bias.shape[1] != nh or not bias.is_contiguous() or bias_edges.numel() != rows
                or not bias_edges.is_contiguous() or not 0 < rows <= 1024):
            raise KernelError("attention: the distance bias is [rows <= 1024, heads] with one "
                              "edge per row")
    if slope is not None:
        _need(slope, "slope", torch.float32, 1)
        if slope.numel() != nh or not slope.is_contiguous():
            raise KernelError("attention: the slope has one number per query head")
    _check(lib().cretif_attn_simt(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _dt(q), _p(kc), _p(vc), _p(table),
        table.stride(0), _p(tok_pos), _p(tok_seq), _p(seq_slot), nh, nkv, hd,
        ctypes.c_float(scale), window, block_tokens, T, _p(sink), vd, _p(bias), _p(bias_edges),
        rows, _p(slope), _stream()), "attn_simt")


# ------------------------------------------------------------------ sampling
def sample(logits, out, temperature: float, top_k: int, seed: int, request=None,
           draw=None, seed_dev=None) -> None:
    """``seed_dev`` (one int64 on the device), when given, is read by the kernel instead of
    ``seed``: a captured launch then serves any seed."""
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    rows, V = logits.shape
    if out.numel() < rows:
        raise KernelError("sample: out is shorter than the number of rows")
    if request is not None:
        _need(request, "request", torch.int64, 1)
    if draw is not None:
        _need(draw, "draw", torch.int32, 1)
    if seed_dev is not None:
        _need(seed_dev, "seed_dev", torch.int64, 1)
    if temperature > 0 and 0 < top_k < V and top_k > lib().cretif_max_top_k():
        raise KernelError(f"sample: top_k {top_k} exceeds the kernel's limit "
                          f"{lib().cretif_max_top_k()}")
    _check(lib().cretif_sample(_p(logits), _rows(logits, "logits"), rows, V,
                               ctypes.c_float(temperature), int(top_k),
                               ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _p(seed_dev),
                               _p(request), _p(draw), _p(out), _stream()), "sample")


def uniform01(seed: int, request: int, draw: int) -> float:
    """The uniform number the sampling kernel uses for (seed, request, draw)."""
    return float(lib().cretif_uniform01(ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF),
                                        ctypes.c_longlong(request), draw))


# ------------------------------------------------------------------ fast products (bfloat16)
def gemv_supported(x, w, out) -> bool:
    """The weight-streaming kernel takes bfloat16 operands with 16-byte aligned rows."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= 64
            and K % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and out.dtype in (torch.bfloat16, torch.float32))


def gemv_bf16(x, w, out, accumulate: bool = False) -> None:
    """out[M,N] (+)= x[M,K] · w[N,K]ᵀ for M <= 64 (decode), tensor-core FMA, 32-bit sums."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemv: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _check(lib().cretif_gemm_skinny(_p(x), _p(w), _p(out), _dt(out), M, N, K, _rows(x, "x"),
                                    _rows(w, "w"), _rows(out, "out"), int(accumulate),
                                    _stream()), "gemm_skinny")


_FAULT = {}


def fault_word(device) -> torch.Tensor:
    """The int32 status word of a device that kernels OR their fault bits into."""
    key = str(torch.device(device))
    if key not in _FAULT:
        _FAULT[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _FAULT[key]


def wait_that_expires(limit: int = 2000, fault=None) -> None:
    """Launch one CTA whose bounded wait runs out after ``limit`` polls: it sets the
    "wait expired" bit of the status word and returns.  Harmless; for exercising the path
    from an expired wait to the host's error."""
    if fault is None:
        fault = fault_word(torch.device("cuda", torch.cuda.current_device()))
    _need(fault, "fault", torch.int32)
    _check(lib().cretif_wait_that_expires(int(limit), _p(fault), None, _stream()),
           "wait_that_expires")


def gemm_tc_supported(x, w, out) -> bool:
    """The tensor-core kernel takes bfloat16 operands whose rows are 16-byte aligned."""
    K = x.shape[1]
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0):
        return False
    if out.dtype == torch.bfloat16:
        return out.stride(0) % 8 == 0
    return out.dtype == torch.float32 and out.stride(0) % 4 == 0


def set_tc_epilogue_warps(n: int) -> int:
    """(For tests that run both.)  Epilogue warps of the tensor-core product: 4 or 8; 0 lets
    each launch choose.  Returns the old setting."""
    return int(lib().cretif_set_tc_epilogue_warps(int(n)))


def gemm_tc(x, w, out, accumulate: bool = False, bn: int = 0, alpha: float = 1.0,
            unary: Optional[str] = None) -> None:
    """out[M,N] (+)= alpha · x[M,K] · w[N,K]ᵀ with TMA, tcgen05.mma and a TMEM accumulator;
    ``unary`` (a key of ACTIVATIONS; stores only) is applied to the 32-bit sums."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _check(lib().cretif_gemm_tc(_p(x), _p(w), _p(out), _dt(out), M, N, K, _rows(x, "x"),
                                _rows(w, "w"), _rows(out, "out"), int(accumulate), bn,
                                ctypes.c_float(alpha),
                                0 if unary is None else 1 + ACTIVATIONS[unary],
                                _p(fault_word(x.device)), _stream()), "gemm_tc")


# ------------------------------------------------------------------ fast attention (bfloat16)
_SM_COUNT = {}


def sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SM_COUNT[key]


def attn_decode_supported(hd: int, block_tokens: int, group: int = 1) -> bool:
    return block_tokens == 64 and hd % 16 == 0 and 16 <= hd <= 256 and group <= 8


def decode_splits(B: int, nkv: int, max_context: int, device) -> int:
    """Ranges per (sequence, kv head): enough CTAs for about four per SM, at most one per
    cache block of the longest context."""
    tiles = max(1, -(-max_context // 64))
    want = (3 * sm_count(device)) // max(1, B * nkv)      # about three CTAs fit an SM: one wave
    return max(1, min(tiles, want, 64))


CLUSTER_MAX_RANGES = 8


def decode_plan(B: int, nkv: int, max_context: int, device, hd: int = 64):
    """(ranges per (sequence, kv head), merge inside a cluster?) for the decode attention.

    Up to eight ranges can be one thread-block cluster, whose merge through distributed
    shared memory is some 5 us shorter than the one through global scratch; a range is a
    cache block or more, and a block costs about 0.3 us.  So the cluster is taken unless it
    would make a CTA walk 16 blocks more than the plain split would (a long context with
    few sequences).  Cluster sizes are powers of two: at batch 16 and 32 of a 3-kv-head model
    clusters of 6 and 3 took 13.8 and 20.0 us against 9.2 and 12.7 us for 4.  A grid beyond two
    CTAs per SM runs with the shallow ring and in more than one wave, which ranges of up to
    sixteen blocks do not pay for (batch 16 with 8 and 4 ranges: 11.0 and 9.2 us at a context
    of 2,100, 14.3 and 11.5 us at 3,000, 16.4 and 13.7 us at 4,000), so a cluster of 8 becomes
    one of 4 there (4 against 2 at batch 32: 12.7 and 14.3 us, so no further).  (Clusters of
    16, which the hardware takes as an opt-in size, were measured: no gain for one sequence,
    twice the time for eight: too few of them fit the chip at once.)"""
    tiles = max(1, -(-max_context // 64))
    n_split = decode_splits(B, nkv, max_context, device)
    if hd > 128 or _decode_simt_only:
        return n_split, False
    n_cluster = max(1, min(n_split, tiles, CLUSTER_MAX_RANGES))
    n_cluster = 1 << (n_cluster.bit_length() - 1)     # clusters of 3, 6 or 7 CTAs place badly
    if n_cluster > 4 and n_cluster * B * nkv > 2 * sm_count(device) and tiles <= 16 * n_cluster:
        n_cluster //= 2
    if -(-tiles // n_cluster) - -(-tiles // n_split) < 16:
        return n_cluster, True
    return n_split, False


def attn_decode(q, out, kc, vc, table, tok_pos, tok_seq, seq_slot, nh: int, nkv: int, hd: int,
                scale: float, window: int, block_tokens: int, n_splits: int, fault,
                cluster: bool = False, sink=None, bias_near=None, bias_far=None,
                head_groups: int = 1, bias_slope=None) -> None:
    """``bias_slope`` (float32 [heads], times log2 e; tensor-core kernel only, not with the
    table): the key n positions back has n times it taken off its scaled score.
    ``head_groups`` = G > 1 (tensor-core kernel only): more than eight query heads on a
    key/value head in ONE launch; the rows of ``q``, ``out``, ``tok_pos`` and ``tok_seq`` are
    (sequence, group of ``nh`` heads) items, G of them a sequence, while ``sink`` and the bias
    keep a row per head of all G·nh.  ``sink`` (float32 [heads], optional; tensor-core kernel only): exp(sink_h) joins head h's
    softmax denominator.  ``bias_near`` [heads, n_far] with ``bias_far`` [heads] (float32, times
    log2 e; tensor-core kernel only): what the key n positions back adds to its scaled score."""
    n_far = 0
    if bias_near is not None:
        _need(bias_near, "bias_near", torch.float32, 2); _need(bias_far, "bias_far", torch.float32, 1)
        n_far = bias_near.shape[1]
        if (bias_near.shape[0] != nh * head_groups or bias_far.numel() != nh * head_groups
                or not bias_near.is_contiguous()
                or not bias_far.is_contiguous() or hd > 128 or _decode_simt_only):
            raise KernelError("attn_decode: the bias is [heads, distances] with one far value "
                              "per head, and needs head_dim <= 128")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.numel() != nh * head_groups or hd > 128 or _decode_simt_only:
            raise KernelError("attn_decode: a sink needs one number per head and head_dim <= 128")
    if bias_slope is not None:
        _need(bias_slope, "bias_slope", torch.float32, 1)
        if (bias_slope.numel() != nh * head_groups or not bias_slope.is_contiguous() or hd > 128
                or _decode_simt_only or bias_near is not None):
            raise KernelError("attn_decode: a slope has one number per head, needs head_dim <= "
                              "128 and comes without a bias table")
    if head_groups > 1 and (hd > 128 or _decode_simt_only or q.shape[0] % head_groups):
        raise KernelError("attn_decode: groups of heads need head_dim <= 128 and whole "
                          "sequences of items")
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(kc, "k cache", torch.bfloat16, 4); _need(vc, "v cache", torch.bfloat16, 4)
    B = q.shape[0]
    if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
            or not vc.is_contiguous()):
        raise KernelError("attn_decode: cache must be contiguous [blocks, kv_heads, 64, head_dim]")
    if n_splits > 64:
        raise KernelError("attn_decode: at most 64 ranges per (sequence, kv head)")
    if cluster:
        if hd > 128 or _decode_simt_only or n_splits > CLUSTER_MAX_RANGES:
            raise KernelError("attn_decode: the cluster merge takes head sizes up to 128 and at "
                              f"most {CLUSTER_MAX_RANGES} ranges")
        _check(lib().cretif_attn_decode_mma_bias(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(kc), _p(vc),
            ctypes.c_longlong(kc.shape[0]), _p(table), table.stride(0), _p(tok_pos), _p(tok_seq),
            _p(seq_slot), nh, nkv, hd, ctypes.c_float(scale), window, block_tokens, B, n_splits,
            None, None, None, _p(sink), _p(bias_near), _p(bias_far), n_far, head_groups,
            _p(bias_slope), _p(fault), _stream()),
            "attn_decode_mma")
        return
    part_o = torch.empty((B, nh, n_splits, hd), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((B, nh, n_splits, 2), dtype=torch.float32, device=q.device)
    counters = _decode_counters(q.device, B * nkv)
    if hd <= 128 and not _decode_simt_only:
        _check(lib().cretif_attn_decode_mma_bias(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(kc), _p(vc),
            ctypes.c_longlong(kc.shape[0]), _p(table), table.stride(0), _p(tok_pos), _p(tok_seq),
            _p(seq_slot), nh, nkv, hd, ctypes.c_float(scale), window, block_tokens, B, n_splits,
            _p(part_o), _p(part_ml), _p(counters), _p(sink), _p(bias_near), _p(bias_far), n_far,
            head_groups, _p(bias_slope), _p(fault), _stream()), "attn_decode_mma")
        return
    _check(lib().cretif_attn_decode(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(kc), _p(vc), _p(table),
        table.stride(0), _p(tok_pos), _p(tok_seq), _p(seq_slot), nh, nkv, hd,
        ctypes.c_float(scale), window, block_tokens, B, n_splits, _p(part_o), _p(part_ml),
        _p(counters), _p(fault), _stream()), "attn_decode")


_COUNTERS = {}
_decode_simt_only = False


def decode_attention_simt_only(on: bool) -> None:
    """Use the CUDA-core decode attention kernel even where the tensor-core one applies
    (it is the only one for head sizes above 128; tests run both)."""
    global _decode_simt_only
    _decode_simt_only = bool(on)


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zeroed int32 counters the decode attention uses to find its last CTA; every launch
    leaves them zero, so one buffer per device serves all launches on a stream."""
    key = str(torch.device(device))
    if key not in _COUNTERS or _COUNTERS[key].numel() < n:
        _COUNTERS[key] = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
    return _COUNTERS[key]


# ------------------------------------------------------------------ fused decode projections
FUSED_MAX_ROWS = 128     # the kernels' limit; the parts choose how far they use it
# Beyond 32 rows the kernels read the matrix once per group of 16 or 32 rows: worth it while
# the matrix is small (measured at 64 tokens: 0.7 of the tensor-core path's time at
# SmolLM2-135M sizes, where no matrix but the head exceeds 4 MB, 0.83 at 360M sizes (up to
# 10 MB), 1.2 at 1.7B sizes (25 to 67 MB)).
FUSED_GROUPS_MAX_BYTES = 16 << 20


def fused_supported(M: int, K: int, w, norm: bool = True) -> bool:
    """Whether the fused kernel takes M rows of width K against w (``norm``: with the norm
    prologue, which keeps the normed rows in shared memory)."""
    if M > 32 and w.numel() * w.element_size() > FUSED_GROUPS_MAX_BYTES:
        return False
    return (w.dtype == torch.bfloat16 and 0 < M <= FUSED_MAX_ROWS and K % 8 == 0
            and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and bool(lib().cretif_fused_smem_ok(M, K, int(norm))))


def set_stream_min_k(k: int, min_bytes: int = -1) -> int:
    """(For tests that must run both variants of the fused product on one shape.)  The fused product streams weights through shared memory for matrices of at least k
    columns or (if not negative) at least min_bytes bytes; returns the old column count."""
    return int(lib().cretif_set_stream_min_k(int(k), ctypes.c_longlong(int(min_bytes))))


def stream_min_bytes() -> int:
    """The size threshold of set_stream_min_k."""
    fn = lib().cretif_stream_min_bytes
    fn.restype = ctypes.c_longlong
    return int(fn())


def set_fused_cluster(n: int) -> int:
    """Largest thread-block cluster that shares the norm prologue of the register variant
    (more than eight rows; 1: none, at most 4); returns the old value."""
    return int(lib().cretif_set_fused_cluster(int(n)))


def set_dependent_launch(on: bool) -> bool:
    """Programmatic dependent launch of the fused kernels on or off; returns the old setting."""
    return bool(lib().cretif_set_dependent_launch(int(on)))


def fused_norm_linear(h, norm_w, eps: float, w, out, rows=None, accumulate: bool = False,
                      unary: Optional[str] = None) -> None:
    """out (+)= bf16(rmsnorm(h[rows])) · wᵀ in one kernel (decode-sized row counts); ``unary``
    (a key of ACTIVATIONS; stores only) is applied to the 32-bit sums."""
    _need(h, "h", torch.float32, 2); _need(norm_w, "norm weight", torch.float32, 1)
    _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    K = h.shape[1]
    M = h.shape[0] if rows is None else rows.numel()
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or not h.is_contiguous():
        raise KernelError("fused_norm_linear: shapes do not fit")
    _check(lib().cretif_fused_linear(None, 0, _p(h), _p(norm_w), _p(rows), ctypes.c_float(eps),
                                     _p(w), _rows(w, "w"), _p(out), _dt(out), _rows(out, "out"),
                                     int(accumulate), ctypes.c_float(1.0),
                                     0 if unary is None else 1 + ACTIVATIONS[unary], M, N, K,
                                     _p(fault_word(h.device)), _stream()), "fused_norm_linear")


def fused_linear_add(x, w, h) -> None:
    """h += x · wᵀ (x bfloat16, h the float32 residual stream)."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2)
    _need(h, "h", torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(h.shape) != (M, N):
        raise KernelError("fused_linear_add: shapes do not fit")
    _check(lib().cretif_fused_linear(_p(x), _rows(x, "x"), None, None, None, ctypes.c_float(0.0),
                                     _p(w), _rows(w, "w"), _p(h), F32, _rows(h, "h"), 1,
                                     ctypes.c_float(1.0), 0, M, N, K,
                                     _p(fault_word(h.device)), _stream()), "fused_linear_add")


def fused_linear_x(x, w, out, accumulate: bool = False, alpha: float = 1.0,
                   unary: Optional[str] = None) -> None:
    """out (+)= alpha · x · wᵀ with the few-token kernels (x bfloat16; out bfloat16, or float32
    which may be added to); ``unary`` (a key of ACTIVATIONS; stores only) is applied to the
    32-bit sums."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError("fused_linear_x: shapes do not fit")
    _check(lib().cretif_fused_linear(_p(x), _rows(x, "x"), None, None, None, ctypes.c_float(0.0),
                                     _p(w), _rows(w, "w"), _p(out), _dt(out), _rows(out, "out"),
                                     int(accumulate), ctypes.c_float(alpha),
                                     0 if unary is None else 1 + ACTIVATIONS[unary], M, N, K,
                                     _p(fault_word(x.device)), _stream()), "fused_linear_x")


def fused_gate_up_silu_x(x, w_gu, act, block: int = 0) -> None:
    """act = silu(x·Wgᵀ) ⊙ (x·Wuᵀ) from bfloat16 rows, one few-token kernel."""
    _need(x, "x", torch.bfloat16, 2); _need(w_gu, "w_gu", torch.bfloat16, 2)
    _need(act, "act", torch.bfloat16, 2)
    M, K = x.shape
    I = act.shape[1]
    if tuple(w_gu.shape) != (2 * I, K) or act.shape[0] != M or not act.is_contiguous():
        raise KernelError("fused_gate_up_silu_x: shapes do not fit")
    _check(lib().cretif_fused_gate_up_silu_x(_p(x), _rows(x, "x"), _p(w_gu), _rows(w_gu, "w_gu"),
                                             _p(act), I, block, M, K, _p(fault_word(x.device)),
                                             _stream()), "fused_gate_up_silu_x")


def fused_qkv_rope(h, norm_w, eps: float, w_qkv, q_out, cos, sin, pairing: int, nh: int,
                   nkv: int, hd: int, tok_pos, tok_seq, seq_slot, table, kc, vc,
                   block_tokens: int, write_cache: bool, fault) -> None:
    """norm → q|k|v product → rotary → q buffer and block cache, one kernel."""
    _need(h, "h", torch.float32, 2); _need(w_qkv, "w_qkv", torch.bfloat16, 2)
    _need(q_out, "q", torch.bfloat16, 2)
    M, K = h.shape
    if w_qkv.shape != ((nh + 2 * nkv) * hd, K) or not h.is_contiguous():
        raise KernelError("fused_qkv_rope: shapes do not fit")
    if cos.shape[1] != hd // 2:
        raise KernelError("fused_qkv_rope: needs rotary_dim == head_dim")
    _check(lib().cretif_fused_qkv_rope(
        _p(h), _p(norm_w), ctypes.c_float(eps), _p(w_qkv), _rows(w_qkv, "w_qkv"), _p(q_out),
        _rows(q_out, "q"), _p(cos), _p(sin), pairing, nh, nkv, hd, _p(tok_pos), _p(tok_seq),
        _p(seq_slot), _p(table), table.stride(0), _p(kc), _p(vc), block_tokens,
        int(write_cache), M, K, _p(fault), _stream()), "fused_qkv_rope")


def fused_gate_up_silu(h, norm_w, eps: float, w_gu, act, block: int = 0) -> None:
    """act = silu(norm(h)·Wgᵀ) ⊙ (norm(h)·Wuᵀ), one kernel; w_gu = [Wg; Wu] stacked
    (``block`` = 0) or with rows interleaved in groups of ``block``."""
    _need(h, "h", torch.float32, 2); _need(w_gu, "w_gu", torch.bfloat16, 2)
    _need(act, "act", torch.bfloat16, 2)
    M, K = h.shape
    I = act.shape[1]
    if tuple(w_gu.shape) != (2 * I, K) or act.shape[0] != M or not act.is_contiguous():
        raise KernelError("fused_gate_up_silu: shapes do not fit")
    _check(lib().cretif_fused_gate_up_silu(_p(h), _p(norm_w), ctypes.c_float(eps), _p(w_gu),
                                           _rows(w_gu, "w_gu"), _p(act), I, block, M, K,
                                           _p(fault_word(h.device)), _stream()),
           "fused_gate_up_silu")


def gemm_tc_silu(x, w_gu, act) -> None:
    """act = silu(x·Wgᵀ) ⊙ (x·Wuᵀ) on the tensor cores; w_gu rows interleaved in groups of 64."""
    _need(x, "x", torch.bfloat16, 2); _need(w_gu, "w_gu", torch.bfloat16, 2)
    _need(act, "act", torch.bfloat16, 2)
    M, K = x.shape
    I = act.shape[1]
    if tuple(w_gu.shape) != (2 * I, K) or act.shape[0] != M or not act.is_contiguous():
        raise KernelError("gemm_tc_silu: shapes do not fit")
    _check(lib().cretif_gemm_tc_silu(_p(x), _p(w_gu), _p(act), M, I, K, _rows(x, "x"),
                                     _rows(w_gu, "w_gu"), _p(fault_word(x.device)), _stream()),
           "gemm_tc_silu")


def gemm_tc_qkv_rope(x, w_qkv, q_out, cos, sin, pairing: int, nh: int, nkv: int, hd: int,
                     tok_pos, tok_seq, seq_slot, table, kc, vc, block_tokens: int,
                     write_cache: bool) -> None:
    """q|k|v product on the tensor cores with rotary and the cache write in its epilogue."""
    _need(x, "x", torch.bfloat16, 2); _need(w_qkv, "w_qkv", torch.bfloat16, 2)
    _need(q_out, "q", torch.bfloat16, 2)
    M, K = x.shape
    if tuple(w_qkv.shape) != ((nh + 2 * nkv) * hd, K) or q_out.shape[0] != M:
        raise KernelError("gemm_tc_qkv_rope: shapes do not fit")
    if cos.shape[1] != hd // 2:
        raise KernelError("gemm_tc_qkv_rope: needs rotary_dim == head_dim")
    _check(lib().cretif_gemm_tc_qkv_rope(
        _p(x), _p(w_qkv), _p(q_out), _rows(q_out, "q"), _p(cos), _p(sin), pairing, nh, nkv, hd,
        _p(tok_pos), _p(tok_seq), _p(seq_slot), _p(table), table.stride(0), _p(kc), _p(vc),
        block_tokens, int(write_cache), M, K, _rows(x, "x"), _rows(w_qkv, "w_qkv"),
        _p(fault_word(x.device)), _stream()), "gemm_tc_qkv_rope")


def set_tc_pair(mode: int) -> int:
    """(For tests that run both.)  The tensor-core product with two CTAs on a tile: -1 where
    the launcher sees fit (the default), 0 never, 1 wherever the kernel takes the product.
    Returns the old setting."""
    return int(lib().cretif_set_tc_pair(int(mode)))


def set_tc_bulk_add(on: bool) -> bool:
    """(For tests that run both.)  Whether the tensor-core product adds into a float32 matrix
    through TMA where it can (the default).  Returns the old setting."""
    return bool(lib().cretif_set_tc_bulk_add(1 if on else 0))


def set_prefill_pairing(mode: int) -> int:
    """(For tests that run all.)  Which prefill attention kernel takes head sizes up to 64
    without a window: -1 as the launcher sees fit (the default), 0 the kernel with two threads
    per row, 1 a thread per row and two query tiles per CTA, 2 a thread per row and one tile
    per CTA whose key steps two groups of warps share.  Returns the old setting."""
    return int(lib().cretif_set_prefill_pairing(int(mode)))


def attn_prefill_supported(hd: int, block_tokens: int) -> bool:
    return block_tokens == 64 and hd % 16 == 0 and 16 <= hd <= 128


def attn_prefill(qkv, out, kc, vc, table, cu_seqlens, seq_start, seq_slot, nh: int, nkv: int,
                 hd: int, scale: float, window: int, block_tokens: int, B: int, max_new: int,
                 fault, sink=None, bias_near=None, bias_far=None, bias_slope=None) -> None:
    """Causal attention of whole prompts; ``qkv`` rows start with the query heads.  ``sink``
    (float32 [heads], optional): exp(sink_h) joins head h's softmax denominator.  ``bias_near``
    [heads, n_far] with ``bias_far`` [heads] (float32, times log2 e): what the key n positions
    back adds to its scaled score, for n < n_far and for every n beyond.  ``bias_slope`` (float32
    [heads], times log2 e; not with the table): n times it is taken off that score instead."""
    n_far = 0
    if bias_near is not None:
        _need(bias_near, "bias_near", torch.float32, 2); _need(bias_far, "bias_far", torch.float32, 1)
        n_far = bias_near.shape[1]
        if (bias_near.shape[0] != nh or bias_far.numel() != nh or not bias_near.is_contiguous()
                or not bias_far.is_contiguous()):
            raise KernelError("attn_prefill: the bias is [heads, distances] with one far value "
                              "per head")
    if bias_slope is not None:
        _need(bias_slope, "bias_slope", torch.float32, 1)
        if bias_slope.numel() != nh or not bias_slope.is_contiguous() or bias_near is not None:
            raise KernelError("attn_prefill: a slope has one number per head and comes without "
                              "a bias table")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.numel() != nh:
            raise KernelError("attn_prefill: the sink has one number per query head")
    _need(qkv, "qkv", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(kc, "k cache", torch.bfloat16, 4); _need(vc, "v cache", torch.bfloat16, 4)
    if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
            or not vc.is_contiguous()):
        raise KernelError("attn_prefill: cache must be contiguous [blocks, kv_heads, 64, head_dim]")
    _check(lib().cretif_attn_prefill_tc_bias(
        _p(qkv), _rows(qkv, "qkv"), qkv.shape[0], _p(out), _rows(out, "out"), _p(kc), _p(vc),
        ctypes.c_longlong(kc.shape[0]), _p(table), table.stride(0), _p(cu_seqlens), _p(seq_start),
        _p(seq_slot), nh, nkv, hd, ctypes.c_float(scale), window, block_tokens, B, max_new,
        _p(sink), _p(bias_near), _p(bias_far), n_far, _p(bias_slope), _p(fault), _stream()),
        "attn_prefill_tc")
