"""A plain, slow Mipurax: whole sequences, no cache, one function per mechanism.

The yardstick for the engine's Mipurax parts.  It shares no code with the package: config.json
is read with ``json``, the weights with the ``safetensors`` library, and everything is
elementary torch arithmetic on the CPU in float64 (or float32).

Notation: ``x`` [S, D] is the residual stream of one sequence of S tokens at positions
0 .. S-1; a linear map is stored [out, in] and applied as ``x @ W.T``;
``unit(x) = x / sqrt(mean(x**2) + eps)`` over the last axis.

* input: ``x = unit(embed[id]) * (1 + n_in)``;
* block: ``x += mixer(unit(x) * (1 + n1))``, then (where the layer has one)
  ``x += ff(unit(x) * (1 + n2))``;
* mixers -- attention through two low-rank latents (one for the queries, one that is all a
  token leaves behind for keys and values, beside a small rotated key part that all heads
  share), with a gate on the output, channel by channel or head by head, and optionally one more
  learned term in the softmax's denominator; and grouped-query attention that sees only the keys
  of its own chunk of positions and takes a multiple of the distance off every score, whose keys
  and values may be those of an earlier layer;
* feed-forward: ``down(gelu(up x))``, alone, or as routed experts: logistic scores, the best
  groups of neighbouring experts, the best experts inside them, the chosen scores divided by
  their sum, plus an expert that every token uses;
* logits: ``(unit(x) * (1 + n_out)) @ embed.T``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

WEIGHT_SUM_EPS = 1e-20      # added to the sum of the chosen experts' scores


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


def norm_around_zero(x, w, eps):
    """The block's norm: the stored weight is the factor's distance from one."""
    return unit(x, eps) * (1.0 + w)


def gelu(z):
    """The exact form, with the error function."""
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def logistic(z):
    return 1.0 / (1.0 + torch.exp(-z))


def rotate(z, base: float, dims: int, layout: str, first_pos: int = 0):
    """z [S, heads, d]: the first ``dims`` channels of every head are rotated by the angle
    p * base^(-2i/dims) for pair i; the rest pass.  ``layout`` says which channels are pair i:
    "interleaved" (2i, 2i+1) or "half" (i, i + dims/2)."""
    S = z.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    ang = (torch.arange(S, dtype=torch.float64) + first_pos)[:, None] * freq[None, :]
    c = torch.cos(ang).to(z.dtype)[:, None, :]
    s = torch.sin(ang).to(z.dtype)[:, None, :]
    out = z.clone()
    if layout == "interleaved":
        u, v = z[..., 0:dims:2], z[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    elif layout == "half":
        u, v = z[..., :half], z[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    else:
        raise ValueError(layout)
    return out


def causal_mask(S: int) -> torch.Tensor:
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    return j <= i


def chunk_mask(S: int, size: int) -> torch.Tensor:
    """visible[i, j]: j <= i and both in the same run of ``size`` positions counted from 0."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    return (j <= i) & (i // size == j // size)


def distance_slopes(heads: int) -> torch.Tensor:
    """Head h takes 2^(-8 (h + 1) / heads) times the distance off its scores."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return 2.0 ** (-8.0 * h / heads)


def softmax_rows(scores, visible, sink=None):
    """scores [H, S, S], visible [S, S]; ``sink`` [H]: exp(sink_h) joins row sums of head h and
    brings nothing else."""
    s = scores.masked_fill(~visible[None], -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None].to(s.dtype))
    p = torch.exp(s - m)
    total = p.sum(dim=-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink[:, None, None].to(s.dtype) - m)
    return p / total


def latent_attention(x, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, layout: str,
                     sink: bool, gate: str):
    """``layout``: pairing of the rotation; ``sink``: the learned term in the denominator;
    ``gate``: "channel" (a logistic gate per output channel) or "head" (one per head)."""
    S = x.shape[0]
    H, d, r, e, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    cq = unit(x @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(S, H, d + r)
    q_flat, q_rot = q[..., :d], rotate(q[..., d:], base, dims, layout)
    ckr = x @ w[p + "dkv"].T
    c = unit(ckr[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate(ckr[:, None, rank:], base, dims, layout)[:, 0]          # [S, r], all heads
    k_flat = (c @ w[p + "uk"].T).view(S, H, d)
    v = (c @ w[p + "uv"].T).view(S, H, e)
    scores = (torch.einsum("ihd,jhd->hij", q_flat, k_flat)
              + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * float(m["scale"])
    pr = softmax_rows(scores, causal_mask(S), w[p + "sink"] if sink else None)
    o = torch.einsum("hij,jhe->ihe", pr, v)
    g = logistic(x @ w[p + "g"].T)
    o = o * (g.view(S, H, e) if gate == "channel" else g.view(S, H, 1))
    return o.reshape(S, H * e) @ w[p + "o"].T


def chunked_attention(x, w, p: str, m: dict, kv=None):
    """Returns (output, (k, v)); ``kv``: keys and values of another layer to use instead of
    projecting them."""
    S = x.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w[p + "q"].T).view(S, H, d)
    if kv is None:
        kv = ((x @ w[p + "k"].T).view(S, G, d), (x @ w[p + "v"].T).view(S, G, e))
    k, v = kv
    kx = k.repeat_interleave(H // G, dim=1)
    vx = v.repeat_interleave(H // G, dim=1)
    i = torch.arange(S, dtype=torch.float64)
    dist = (i[:, None] - i[None, :])
    scores = torch.einsum("ihd,jhd->hij", q, kx) * float(m["scale"]) \
        - distance_slopes(H).to(x.dtype)[:, None, None] * dist.to(x.dtype)[None]
    pr = softmax_rows(scores, chunk_mask(S, int(m["mask"]["size"])))
    o = torch.einsum("hij,jhe->ihe", pr, vx)
    return o.reshape(S, H * e) @ w[p + "o"].T, kv


def dense_ff(x, w, p: str):
    return gelu(x @ w[p + "up"].T) @ w[p + "down"].T


def route(x, router_w, r: dict):
    """(chosen [S, top] expert numbers, weights [S, top]) for rows x."""
    E, top = int(r["experts"]), int(r["top"])
    s = logistic(x @ router_w.T)                               # [S, E]
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups and int(groups["count"]) > 1:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        sg = s.view(-1, n, per)
        best2 = sg.topk(min(2, per), dim=-1).values.sum(dim=-1)        # [S, n]
        kept = best2.topk(keep, dim=-1).indices
        ok = torch.zeros_like(best2, dtype=torch.bool)
        ok.scatter_(1, kept, True)
        allowed = ok[:, :, None].expand(-1, n, per).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + WEIGHT_SUM_EPS)


def routed_ff(x, w, p: str, mlp: dict):
    chosen, weights = route(x, w[p + "router"], mlp["router"])
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for c in range(chosen.shape[1]):
            e = int(chosen[t, c])
            out[t] += weights[t, c] * dense_ff(x[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + dense_ff(x, w, p + "shared.")
    return out


def feed_forward(x, w, p: str, mlp: dict):
    if mlp.get("kind", "dense") == "dense":
        return dense_ff(x, w, p)
    return routed_ff(x, w, p, mlp)


def mixer(i: int, layer: dict, x, w, eps: float, kept: Dict[int, tuple]):
    """``kept``: keys and values of the chunked attention layers so far, by layer."""
    p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
    if kind == "latent_attention":
        return latent_attention(x, w, p, m, eps, "interleaved", sink=False, gate="channel")
    if kind == "latent_attention_2":
        return latent_attention(x, w, p, m, eps, "half", sink=True, gate="head")
    if kind == "attention":
        src = m.get("kv_from")
        y, kv = chunked_attention(x, w, p, m, kv=None if src is None else kept[int(src)])
        kept[i] = kv
        return y
    raise ValueError(kind)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            streams: Optional[list] = None) -> torch.Tensor:
    """Logits [S, vocab] of one sequence; ``streams`` collects the stream after every layer."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = norm_around_zero(w["embed"][torch.tensor(ids, dtype=torch.long)], w["embed.norm"], eps)
    kept: Dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        x = x + mixer(i, layer, norm_around_zero(x, w[f"l{i}.norm1"], eps), w, eps, kept)
        if layer.get("mlp") is not None:
            x = x + feed_forward(norm_around_zero(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp.",
                                 layer["mlp"])
        if streams is not None:
            streams.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T


def greedy(cfg, w, prompt: List[int], n_new: int, dtype=torch.float64) -> List[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(forward(cfg, w, ids, dtype)[-1].argmax()))
    return ids[len(prompt):]
