"""A plain, slow Virorax: whole sequences, no cache, one function per mechanism.

The yardstick for the engine's Virorax parts.  It shares no code with the package: config.json
is read with ``json``, the weights with the ``safetensors`` library, and everything is
elementary torch arithmetic on the CPU in float64 (or float32).

Notation: ``x`` [S, D] is the residual stream of one sequence of S tokens at positions
0 .. S-1; a linear map is stored [out, in] and applied as ``x @ W.T``;
``unit(x) = x / sqrt(mean(x**2) + eps)`` over the last axis.

* input: ``x = embed[id] + pos[p]``;
* block: ``x += m * mixer(unit(x) * n1)``, then (where the layer has one)
  ``x += m * ff(unit(x) * n2)`` with one factor ``m`` for the whole model;
* two mixers -- grouped-query attention with biases, a norm per head on queries and keys, a
  rotation of part of each head, a sliding window, a learned per-head term in the softmax's
  denominator and a per-head output gate; and retention, a matrix-valued recurrence with a fixed
  decay per head;
* feed-forward: ``down(relu(up x) ** 2)``;
* a span of layers runs several times over with the same tensors; before every pass but the
  first the input ``x`` of layer 0 is added to the stream again;
* logits: ``cap * tanh((unit(x) * final) @ embed.T / cap)``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List

import torch


def read_model_folder(model_dir: str):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(torch.float64)
    return cfg, weights


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


def rotate_front(z, base: float, dims: int, first_pos: int = 0):
    """z [S, heads, d]: the first ``dims`` channels of every head are rotated, channel i paired
    with channel i + dims/2, by the angle p * base^(-2i/dims); the rest pass."""
    S = z.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    ang = (torch.arange(S, dtype=torch.float64) + first_pos)[:, None] * freq[None, :]
    c = torch.cos(ang).to(z.dtype)[:, None, :]
    s = torch.sin(ang).to(z.dtype)[:, None, :]
    u, v = z[..., :half], z[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, z[..., dims:]], dim=-1)


def window_mask(S: int, size: int) -> torch.Tensor:
    """visible[i, j]: 0 <= i - j < size."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    return (i - j >= 0) & (i - j < size)


def softmax_with_sink(s, visible, sink):
    """Rows of ``s`` [S, S] over the visible keys, with exp(sink) as one more term of the
    denominator that has no value."""
    s = s.masked_fill(~visible, -math.inf)
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink.expand(s.shape[0], 1))
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - m))


def mixer_attention(h, W, p, m, eps):
    S = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(S, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(S, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(S, G, e)
    q = unit(q, eps) * W[p + "q.norm"]
    k = unit(k, eps) * W[p + "k.norm"]
    q = rotate_front(q, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_front(k, m["rot"]["base"], m["rot"]["dims"])
    vis = window_mask(S, (m.get("mask") or {}).get("size", S))     # no mask: every earlier key
    gate = torch.sigmoid(h @ W[p + "g"].T)                   # [S, H]
    out = torch.zeros(S, H, e, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        w = softmax_with_sink((q[:, hh] @ k[:, g].T) * m["scale"], vis, W[p + "sink"][hh])
        out[:, hh] = (w @ v[:, g]) * gate[:, hh:hh + 1]
    return out.reshape(S, H * e) @ W[p + "o"].T


def retention(q, k, v, decay):
    """q, k [S, H, d], v [S, H, e], decay [H] -> o [S, H, e]; a state M [d, e] per head, zero
    at the start: M <- decay_h M + k v^T; o = M^T q."""
    S, H, d = q.shape
    o = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    for hh in range(H):
        M = torch.zeros(d, v.shape[-1], dtype=q.dtype)
        for t in range(S):
            M = decay[hh] * M + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = M.T @ q[t, hh]
    return o


def mixer_retention(h, W, p, m, eps):
    S = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = rotate_front((h @ W[p + "q"].T).reshape(S, H, d), m["rot"]["base"], m["rot"]["dims"])
    k = rotate_front((h @ W[p + "k"].T).reshape(S, H, d), m["rot"]["base"], m["rot"]["dims"])
    k = k * d ** -0.5
    v = (h @ W[p + "v"].T).reshape(S, H, e)
    o = retention(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = unit(o, eps).reshape(S, H * e) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


MIXERS = {"attention": mixer_attention, "retention": mixer_retention}


def feed_forward(h, W, p):
    return relu_squared(h @ W[p + "up"].T) @ W[p + "down"].T


def layer_order(cfg) -> List[tuple]:
    """(layer, whether a new pass of the repeated span starts here and is not the first)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            streams=None) -> torch.Tensor:
    """Logits [S, vocab] of one whole sequence.  ``streams``, a list, receives the residual
    stream after every layer run."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = torch.stack([W["embed"][t] + W["pos"][p] for p, t in enumerate(ids)])
    x0 = x.clone()
    for i, again in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if again:
            x = x + x0
        y = MIXERS[layer["type"]](unit(x, eps) * W[p + "norm1"], W, p + "mix.", layer["mixer"], eps)
        x = x + mult * y
        if layer.get("mlp") is not None:
            x = x + mult * feed_forward(unit(x, eps) * W[p + "norm2"], W, p + "mlp.")
        if streams is not None:
            streams.append(x.clone())
    logits = (unit(x, eps) * W["final.norm"]) @ W["embed"].T
    cap = cfg.get("logit_softcap")
    return soft_cap(logits, cap) if cap else logits


def greedy(cfg, weights, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        logits = forward(cfg, weights, ids, dtype)[-1]
        best = int(torch.nonzero(logits == logits.max())[0])
        out.append(best)
        ids.append(best)
    return out
