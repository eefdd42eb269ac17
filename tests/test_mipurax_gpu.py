"""Mipurax through the engine against the plain implementation (``plain_mipurax``): every
mechanism alone, every way of cutting requests into steps, chunks' edges, far keys, reused
slots, greedy generation through the library's own entry point."""
import json
import os

import numpy as np
import pytest
import torch

import mipurax_tiny as tiny
import plain_mipurax as plain
from replay_cuts import (rel_err, run_batch, run_chunks, run_schedule, run_tail_by_one,
                         run_whole)

pytestmark = pytest.mark.gpu

# Relative to the largest plain logit.  The float32 runs are the sharp ones; bfloat16 rounds
# activations, keys and values to eight bits several times a layer, so its bound is on the mean
# over the positions with a loose one on the worst.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
BF16_WORST = 0.3


def close(got, want, dtype):
    if dtype == "float32":
        return rel_err(got, want) <= TOL[dtype]
    want = np.asarray(want, dtype=np.float64)
    per_row = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=-1) / np.abs(want).max()
    if len(per_row) < 4:
        return per_row.max() <= BF16_WORST
    return per_row.mean() <= TOL[dtype] and per_row.max() <= BF16_WORST


LENGTHS = {"A": [1, 2, 3, 10, 23, 75, 140], "B": [1, 5, 64, 65, 131, 200], "C": [1, 2, 9, 40],
           "D": [1, 4, 31, 70, 100]}
WIDE = (".dq", ".uq", ".dkv", ".uk", ".uv", ".q", ".k", ".v", ".g", ".o", ".up", ".down")


def _write(tmp_path_factory, name, cfg, seed, edit=None):
    """A model folder for ``cfg`` with seeded random weights; ``edit(tensors)`` may change
    tensors before they are written."""
    from cretif_b200.config import build_mipurax_spec, mipurax_config_from_dict
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights.loader import random_weights, write_model_folder
    d = str(tmp_path_factory.mktemp(f"mipurax_{name}"))
    names, _ = manifest(build_mipurax_spec(mipurax_config_from_dict(cfg)))
    tensors = random_weights(names, seed, torch.bfloat16)
    # wider projections than the default draw: scores, gates and sinks that are not all alike;
    # a quieter router: logits of a few units, so that no two logistic scores round to the same
    # 32-bit number and no choice of experts or groups is a close call
    for k in tensors:
        if k.endswith(WIDE) or k == "embed":
            tensors[k] = (tensors[k].float() * 4.0).to(torch.bfloat16)
        elif k.endswith(".router"):
            tensors[k] = (tensors[k].float() * 0.25).to(torch.bfloat16)
    if edit is not None:
        edit(tensors)
    write_model_folder(d, cfg, tensors)
    return d


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: _write(tmp_path_factory, n, c, tiny.SEEDS[n]) for n, c in tiny.CONFIGS.items()}


@pytest.fixture(scope="module")
def engines(folders):
    from cretif_b200.engine import Engine
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(folders[name], dtype=dtype, max_tokens=max_tokens)
        return made[key]
    return get


@pytest.fixture(scope="module")
def plain_logits(folders):
    models, memo = {}, {}

    def get(name, toks):
        key = (name, tuple(toks))
        if key not in memo:
            if name not in models:
                models[name] = plain.read_model_folder(folders[name])
            cfg, w = models[name]
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        return memo[key]
    return get


# ------------------------------------------------------------------ registry and loading
def test_the_configuration_picks_the_model_and_its_parts(folders):
    from cretif_b200.config import load_config
    from cretif_b200.engine import Engine
    arch, cfg, spec = load_config(folders["A"])
    assert arch.name == "Mipurax" and spec.vocab_size == 96 and spec.hidden_size == 64
    eng = Engine(folders["A"], dtype="float32", max_tokens=256)
    groups = eng.cache.stats()["groups"]
    # two latents (24 + 8 and 48 + 16 wide, one head each) and ONE grouped-query cache: the
    # last layer reads layer 1's
    assert sorted((g["head_dim"], g["layers"], g["window"]) for g in groups) == \
        [(16, 1, 0), (32, 1, 0), (64, 1, 0)]


# ------------------------------------------------------------------ kernels of the mechanisms
def test_exact_gelu_and_a_gate_per_channel():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    x = torch.randn(37, 50, generator=g) * 3
    out = torch.empty(37, 50, device="cuda")
    ops.activation(x.cuda(), out, "gelu")
    assert (out.cpu().double() - plain.gelu(x.double())).abs().max() < 1e-5
    tanh_form = 0.5 * x.double() * (1 + torch.tanh((2 / torch.pi) ** 0.5
                                                  * (x.double() + 0.044715 * x.double() ** 3)))
    assert (plain.gelu(x.double()) - tanh_form).abs().max() > 1e-4       # not the other gelu
    for width, dt in ((50, torch.float32), (50, torch.bfloat16), (48, torch.bfloat16)):
        o = (torch.randn(21, width, generator=g) * 2).to(dt)
        gates = torch.randn(21, width + 8, generator=g) * 2
        want = o.double() * plain.logistic(gates.double()[:, :width])
        oc = o.cuda()
        ops.gate_heads(oc, gates.cuda(), width, 1)
        tol = 1e-5 if dt == torch.float32 else 2.0 ** -7
        assert ((oc.cpu().double() - want).abs() <= tol * want.abs() + 1e-6).all(), (width, dt)


def test_norm_of_the_embedded_rows():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    for R, H in ((1, 40), (19, 64), (300, 257)):
        x = torch.randn(R, H, generator=g) * 5
        w = torch.randn(H, generator=g) * 0.3
        want = plain.norm_around_zero(x.double(), w.double(), 1e-5)
        xc = x.cuda()
        ops.rmsnorm_rows(xc, (w + 1.0).cuda(), 1e-5)
        assert (xc.cpu().double() - want).abs().max() < 1e-5, (R, H)


def _cache_for(positions, nkv, hd, dtype, bt=64):
    n_blocks = (positions + bt - 1) // bt + 1
    kc = torch.zeros(n_blocks, nkv, bt, hd, dtype=dtype, device="cuda")
    table = torch.arange(1, n_blocks + 1, dtype=torch.int32, device="cuda").flip(0)[None, :] - 1
    return kc, table.contiguous()


def _gather(cache, table, positions, bt=64):
    t = table[0].cpu()
    return torch.stack([cache[t[p // bt], :, p % bt].cpu() for p in range(positions)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,rot,rank,q_rank,layout,dims", [
    (2, 16, 8, 24, 40, "interleaved", 8), (4, 8, 16, 48, 24, "half", 16),
    (1, 4, 2, 8, 8, "half", 2), (3, 12, 6, 20, 28, "interleaved", 6),
    (2, 32, 64, 64, 96, "half", 64), (1, 8, 130, 300, 5, "half", 130),
    (2, 8, 16, 24, 16, "half", 6), (3, 4, 12, 16, 8, "interleaved", 4)])
def test_the_latents_their_norms_the_rotated_part_and_the_cache_write(dtype, H, d, rot, rank,
                                                                      q_rank, layout, dims):
    """The kernels between a latent attention's input product and its scores, over a sequence
    fed in pieces (the long piece takes the kernels' many-token forms), against the plain
    functions."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.position import rotary_table
    g = torch.Generator().manual_seed(4)
    S, base, eps = 300, 300.0, 1e-5
    proj = torch.randn(S, q_rank + rank + rot + 5, generator=g) * 2
    wq, wc = torch.randn(q_rank, generator=g), torch.randn(rank, generator=g)
    P = proj.double()
    cq = plain.unit(P[:, :q_rank], eps) * wq.double()
    c = plain.unit(P[:, q_rank:q_rank + rank], eps) * wc.double()
    kr = plain.rotate(P[:, None, q_rank + rank:q_rank + rank + rot], base, dims, layout)[:, 0]
    cos, sin = rotary_table(base, dims, S, torch.device("cuda"))
    pairing = 1 if layout == "interleaved" else 0
    kc, table = _cache_for(S, 1, rank + rot, dtype)
    cq_out = torch.zeros(S, q_rank, dtype=dtype, device="cuda")
    fault = torch.zeros(1, dtype=torch.int32, device="cuda")
    at = 0
    for n in (1, 2, 30, 1, 266):
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        zeros = torch.zeros(n, dtype=torch.int32, device="cuda")
        ops.latent_in(proj[at:at + n].cuda(), q_rank, rank, rot, wq.cuda(), wc.cuda(), eps, cos,
                      sin, pairing, pos, zeros, zeros[:1], cq_out[at:at + n], table=table, kc=kc,
                      fault=fault, rot_dims=dims)
        at += n
    assert at == S and int(fault.item()) == 0
    tol = 1e-4 if dtype == torch.float32 else 6e-2
    rows = _gather(kc, table, S)[:, 0].double()
    assert (cq_out.cpu().double() - cq).abs().max() < tol
    assert (rows[:, :rank] - c).abs().max() < tol
    assert (rows[:, rank:] - kr).abs().max() < tol
    # the queries' rotated parts go behind the latent-space parts
    q = (torch.randn(S, H * (d + rot), generator=g) * 2).to(dtype)
    q_lat = torch.zeros(S, H, rank + rot, dtype=dtype, device="cuda")
    pos = torch.arange(S, dtype=torch.int32, device="cuda")
    ops.rope_heads(q.cuda(), H, d, rot, cos, sin, pairing, pos, q_lat, rank, rot_dims=dims)
    want = plain.rotate(q.double().view(S, H, d + rot)[..., d:], base, dims, layout)
    assert (q_lat[:, :, rank:].cpu().double() - want).abs().max() < tol
    assert bool((q_lat[:, :, :rank] == 0).all())
    few = torch.zeros(40, H, rank + rot, dtype=dtype, device="cuda")
    ops.rope_heads(q[200:240].cuda(), H, d, rot, cos, sin, pairing, pos[200:240], few, rank,
                   rot_dims=dims)
    assert torch.equal(few, q_lat[200:240])


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (12, 2, 4, 3), (6, 3, 2, 2),
                                               (4, 2, 4, 3), (3, 1, 0, 0), (1, 1, 1, 1),
                                               (64, 6, 8, 3), (256, 8, 16, 4), (40, 5, 0, 0)])
def test_routing_with_groups(E, top, groups, keep):
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(E + top)
    T, H = 70, 48
    x = torch.randn(T, H, generator=g)
    router = torch.randn(E, H, generator=g) * 0.4
    rule = {"experts": E, "top": top}
    if groups:
        rule["groups"] = {"count": groups, "keep": keep}
    chosen, weights = plain.route(x.double(), router.double(), rule)
    for way in ("route", "topk"):
        ids = torch.zeros(T, top, dtype=torch.int32, device="cuda")
        wts = torch.zeros(T, top, dtype=torch.float32, device="cuda")
        if way == "route":
            ops.moe_route(x.cuda(), router.cuda(), top, ids, wts, renorm=True, groups=groups,
                          keep=keep, sum_eps=1e-20)
        else:
            logits = (x.double() @ router.double().T).float().cuda()
            ops.moe_topk(logits, top, ids, wts, renorm=True, groups=groups, keep=keep,
                         sum_eps=1e-20)
        for t in range(T):
            got = dict(zip(ids[t].tolist(), wts[t].tolist()))
            want = dict(zip(chosen[t].tolist(), weights[t].tolist()))
            assert set(got) == set(want), (way, t)
            assert all(abs(got[e] - want[e]) < 1e-5 for e in want), (way, t)


def _attention_case(H, G, d, chunk, S, seed):
    """Queries, keys and values with a key that stands out at the first position of every chunk
    (the last one a later query still sees) and one just before it (the first it does not)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, H, d, generator=g)
    k = torch.randn(S, G, d, generator=g)
    for i in range(S):
        q[i, :, 0] += 2.0
    for p in range(0, S, chunk):
        k[p, :, 0] += 3.0
        if p:
            k[p - 1, :, 0] += 4.0
    v = torch.randn(S, G, d, generator=g)
    return q, k, v


def _plain_chunked(q, k, v, chunk, scale, slopes):
    S, H, d = q.shape
    G = k.shape[1]
    i = torch.arange(S, dtype=torch.float64)
    vis = plain.chunk_mask(S, chunk)
    out = torch.zeros(S, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale \
            - slopes[h] * (i[:, None] - i[None, :])
        out[:, h] = plain.softmax_rows(s[None], vis)[0] @ v[:, h // (H // G)].double()
    return out.reshape(S, -1)


@pytest.mark.parametrize("H,G,d,chunk", [(4, 2, 64, 100), (2, 1, 128, 64), (8, 2, 32, 65),
                                         (3, 3, 16, 129), (2, 2, 64, 1), (16, 1, 64, 100),
                                         (24, 2, 32, 70), (12, 1, 48, 33)])
def test_attention_kernels_with_chunks_and_a_slope(H, G, d, chunk):
    """The attention kernels the engine picks in bfloat16 (prompt, portion, single tokens) and
    the plain kernel in float32, with a chunked mask and a slope by distance, against the plain
    softmax on the same inputs."""
    from cretif_b200.parts.attention import run_attention
    from cretif_b200.parts.base import StepContext
    S = 333
    q, k, v = _attention_case(H, G, d, chunk, S, 7)
    slopes = plain.distance_slopes(H)
    scale = 0.7 / d ** 0.5
    dev = torch.device("cuda")
    i32 = dict(dtype=torch.int32, device=dev)
    fault = torch.zeros(1, **i32)
    for dtype in (torch.float32, torch.bfloat16):
        qd, kd, vd = q.to(dtype), k.to(dtype), v.to(dtype)
        want = _plain_chunked(qd, kd, vd, chunk, scale, slopes)
        kc, table = _cache_for(S, G, d, dtype)
        vc = torch.zeros_like(kc)
        t = table[0].cpu()
        for p in range(S):
            kc[t[p // 64], :, p % 64] = kd[p].cuda()
            vc[t[p // 64], :, p % 64] = vd[p].cuda()

        class KV:
            pass
        kv = KV()
        kv.k, kv.v, kv.table, kv.block_tokens, kv.window = kc, vc, table, 64, 0
        slope = slopes.float().cuda()
        tilt = (slopes * 1.4426950408889634).float().cuda()

        def ctx(T, first, decode):
            return StepContext(T=T, B=1, tok_ids=torch.zeros(T, **i32),
                               tok_pos=torch.arange(first, first + T, **i32),
                               tok_seq=torch.zeros(T, **i32), seq_slot=torch.zeros(1, **i32),
                               seq_start=torch.tensor([first], **i32),
                               cu_seqlens=torch.tensor([0, T], **i32), is_decode=decode,
                               max_new=T, max_context=512 if decode else first + T, fault=fault,
                               dtype=dtype, device=dev)
        for first, T, decode in ((0, S, False), (200, S - 200, False), (S - 1, 1, True),
                                 (chunk * (150 // chunk), 1, True), (150, 1, True)):
            out = torch.zeros(T, H * d, dtype=dtype, device=dev)
            run_attention(qd[first:first + T].reshape(T, H * d).cuda(), out,
                          ctx(T, first, decode), kv, H, G, d, scale, -chunk, dtype, None,
                          slope=slope, slope_log2e=tilt)
            err = (out.cpu().double() - want[first:first + T]).abs().max()
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert err <= tol * want.abs().max(), (dtype, first, T, decode, float(err))
    assert int(fault.item()) == 0


@pytest.mark.parametrize("H,d,B", [(16, 96, 1), (32, 128, 3), (24, 64, 2), (12, 48, 2)])
def test_many_heads_on_one_key_value_head_decode(H, d, B):
    """Single tokens of B sequences of unequal length over one shared key/value head whose
    values are its keys (a cached latent), with a sink per head: groups of eight heads go in one
    launch where the head count allows, else eight at a time; both against the plain softmax."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.attention import run_attention
    from cretif_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(H + d)
    lens = [150, 77, 201][:B]
    dev = torch.device("cuda")
    i32 = dict(dtype=torch.int32, device=dev)
    n_blocks = sum((n + 63) // 64 for n in lens) + 1
    kc = torch.zeros(n_blocks, 1, 64, d, dtype=torch.bfloat16, device=dev)
    table = torch.full((B, 8), -1, **i32)
    ks, at = [], 0
    for b, n in enumerate(lens):
        k = torch.randn(n, d, generator=g).bfloat16()
        ks.append(k)
        for p in range(n):
            if p % 64 == 0:
                table[b, p // 64] = n_blocks - 1 - at
                at += 1
            kc[int(table[b, p // 64]), 0, p % 64] = k[p].cuda()
    q = (torch.randn(B, H, d, generator=g) * 1.5).bfloat16()
    sink = torch.randn(H, generator=g) * 2
    scale = 0.8 / d ** 0.5
    want = torch.zeros(B, H, d, dtype=torch.float64)
    for b, n in enumerate(lens):
        s = torch.einsum("hd,jd->hj", q[b].double(), ks[b].double()) * scale
        w = plain.softmax_rows(s[:, None, :], torch.ones(1, n, dtype=torch.bool), sink.double())
        want[b] = w[:, 0] @ ks[b].double()

    class KV:
        pass
    kv = KV()
    kv.k, kv.v, kv.table, kv.block_tokens, kv.window = kc, kc, table, 64, 0
    fault = torch.zeros(1, **i32)
    ctx = StepContext(T=B, B=B, tok_ids=torch.zeros(B, **i32),
                      tok_pos=torch.tensor([n - 1 for n in lens], **i32),
                      tok_seq=torch.arange(B, **i32), seq_slot=torch.arange(B, **i32),
                      seq_start=torch.tensor([n - 1 for n in lens], **i32),
                      cu_seqlens=torch.arange(B + 1, **i32), is_decode=True, max_new=1,
                      max_context=512, fault=fault, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(B, H * d, dtype=torch.bfloat16, device=dev)
    before = ops.launch_count()
    run_attention(q.reshape(B, H * d).cuda(), out, ctx, kv, H, 1, d, scale, 0, torch.bfloat16,
                  sink.cuda())
    launches = ops.launch_count() - before
    assert launches == (1 if H % 8 == 0 else -(-H // 8)), launches
    err = (out.cpu().double() - want.reshape(B, H * d)).abs().max()
    assert err <= 2e-2 * want.abs().max(), float(err)
    assert int(fault.item()) == 0


# ------------------------------------------------------------------ each mechanism alone in a model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "latent_attention", "latent_attention_2"])
def test_one_layer_of_each_mixer(tmp_path_factory, kind, dtype):
    from cretif_b200.engine import Engine
    cfg = tiny.one_layer(kind)
    d = _write(tmp_path_factory, "one_" + kind, cfg, seed=9)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    pcfg, w = plain.read_model_folder(d)
    rng = np.random.default_rng(3)
    for n in (1, 2, 13, 90):
        toks = rng.integers(0, cfg["vocab"], size=n).tolist()
        want = plain.forward(pcfg, w, toks).numpy()
        assert close(run_whole(eng, toks), want, dtype), (kind, n)
        assert close(run_tail_by_one(eng, toks, tail=n), want, dtype), (kind, n)
        assert close(run_chunks(eng, toks, [2, 5, 2, 30]), want, dtype), (kind, n)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mlp", [tiny._ff(72), tiny._moe(8, 2, 40, groups=(4, 2), shared=24),
                                 tiny._moe(5, 3, 64), tiny._moe(4, 1, 8, groups=(2, 1))])
def test_each_feed_forward_through_every_product(tmp_path_factory, mlp, dtype):
    """One attention layer and a feed-forward: steps of a few tokens (an expert's rows streamed
    per pair), of hundreds (rows sorted by expert: tensor cores in bfloat16, 32-bit FMA in
    float32), and the sorted way for few tokens as well."""
    from cretif_b200.engine import Engine
    from cretif_b200.parts.experts import few_pairs_off
    cfg = tiny.one_layer("attention", mlp=mlp)
    d = _write(tmp_path_factory, "ff", cfg, seed=10)
    eng = Engine(d, dtype=dtype, max_tokens=1024, step_graphs=False)
    pcfg, w = plain.read_model_folder(d)
    rng = np.random.default_rng(5)
    toks = rng.integers(0, cfg["vocab"], size=300).tolist()
    want = plain.forward(pcfg, w, toks).numpy()
    assert close(run_whole(eng, toks), want, dtype)
    assert close(run_chunks(eng, toks, [3, 1, 40, 7, 1, 1]), want, dtype)
    try:
        few_pairs_off(True)
        assert close(run_chunks(eng, toks[:30], [3, 1, 20, 1]), want[:30], dtype)
    finally:
        few_pairs_off(False)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_the_stream_after_every_layer(engines, folders, name):
    eng = engines(name, "float32")
    pcfg, w = plain.read_model_folder(folders[name])
    toks = tiny.tokens(name, 19, 7)
    want = []
    plain.forward(pcfg, w, toks, streams=want)
    got = []
    slot = eng.alloc_slot()
    eng.step([(slot, toks)], "all", streams=got)
    eng.free_slot(slot)
    assert len(got) == len(want) == len(eng.spec.schedule)
    for i, (a, b) in enumerate(zip(got, want)):
        assert (a.cpu().double() - b).abs().max() <= 1e-4 * float(b.abs().max()), (name, i)


# ------------------------------------------------------------------ ways of cutting the work
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_and_token_by_token(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    for n in LENGTHS[name]:
        toks = tiny.tokens(name, n, 1)
        want = plain_logits(name, toks)
        got = run_whole(eng, toks)
        assert got.shape == want.shape
        assert close(got, want, dtype), (name, n)
        assert close(run_tail_by_one(eng, toks, tail=32), want, dtype), (name, n)
    toks = tiny.tokens(name, 20, 2)                    # nothing but single tokens
    assert close(run_tail_by_one(eng, toks, tail=20), plain_logits(name, toks), dtype)
    eng.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_few_token_steps_with_and_without_the_fused_kernels(folders, plain_logits, name):
    """bfloat16 steps of a few tokens norm the rows inside the mixers' input products and apply
    the feed-forward's activation in the products' epilogues; with the few-token kernels switched
    off the same steps take the separate kernels.  Both ways give the plain implementation's
    logits, and each other's up to the order of summation."""
    from cretif_b200.csrc import ops
    from cretif_b200.engine import Engine
    from cretif_b200.parts.attention import enable_fused_steps
    eng = Engine(folders[name], dtype="bfloat16", max_tokens=512, step_graphs=False)
    toks = tiny.tokens(name, 40, 7)
    want = plain_logits(name, toks)
    got = {}
    try:
        for on in (True, False):
            enable_fused_steps(on)
            before = ops.launch_count()
            got[on] = run_chunks(eng, toks, [3, 1, 1, 5, 2, 1, 27])
            launches = ops.launch_count() - before
            assert close(got[on], want, "bfloat16"), (name, on)
            got[on] = (got[on], launches)
    finally:
        enable_fused_steps(True)
    assert got[True][1] < got[False][1]                 # fewer kernels the fused way
    assert rel_err(got[True][0], got[False][0]) < 3e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_a_prompt(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    n = LENGTHS[name][-1]
    toks = tiny.tokens(name, n, 3)
    want = plain_logits(name, toks)
    for cuts in ([2, 2, 2, 2], [63, 2, 64], [1, 70, 1, 2], [5] * 12, [n - 2, 2]):
        assert close(run_chunks(eng, toks, cuts), want, dtype), (name, cuts)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_unequal_batches_against_each_alone_and_reused_slots(engines, plain_logits, name, dtype):
    """Batches of unequal requests on a cache too small for two batches: the second and third
    rounds get slots and blocks that were used before."""
    eng = engines(name, dtype, max_tokens=640)
    lens = LENGTHS[name]
    for round_ in range(3):
        reqs = [tiny.tokens(name, n + 6 + 2 * i, 20 + round_) for i, n in enumerate(lens[:5])]
        prompts = [min(lens[i], len(r)) for i, r in enumerate(reqs)]
        outs = run_batch(eng, reqs, prompts)
        for r, got in zip(reqs, outs):
            assert close(got, plain_logits(name, r), dtype), (name, round_, len(r))
        eng.cache.check()
        assert eng.cache.stats()["slots_live"] == 0
    # a mixture: fresh prompts, further portions and single tokens in the same steps
    reqs = [tiny.tokens(name, n, 30) for n in (40, 9, 27)]
    outs = run_schedule(eng, reqs, [[(0, 18)], [(0, 2), (1, 9)], [(0, 1), (2, 25)],
                                    [(0, 19), (2, 2)]])
    for r, got in zip(reqs, outs):
        assert close(got, plain_logits(name, r), dtype), name
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_chunk(engines, plain_logits, dtype):
    """A short prompt and then 230 single tokens: both chunk sizes of B (130 and 70 keys) start
    anew among decoded tokens, away from block borders."""
    eng = engines("B", dtype)
    toks = tiny.tokens("B", 240, 5)
    got = run_tail_by_one(eng, toks, tail=230)
    assert close(got, plain_logits("B", toks), dtype)
    eng.cache.check()


# ------------------------------------------------------------------ what a position may depend on
def _one_layer_engine(tmp_path_factory, kind, mixer, edit=None, dtype="float32", mlp=None):
    from cretif_b200.engine import Engine
    cfg = tiny.one_layer(kind, mixer=mixer, mlp=mlp)
    d = _write(tmp_path_factory, f"edge_{kind}", cfg, seed=13, edit=edit)
    return Engine(d, dtype=dtype, max_tokens=2048), plain.read_model_folder(d), cfg


@pytest.mark.parametrize("chunk", [1, 7, 64, 65, 129])
def test_a_chunk_begins_where_it_should(tmp_path_factory, chunk):
    """One attention layer alone: the logits at position i depend on the tokens from the start of
    i's chunk to i and on nothing else.  Changing the chunk's first token changes them, changing
    the token before it does not, for a position inside a prompt and for a decoded one."""
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention",
                                            tiny._att(4, 2, 16, 16, chunk, 0.25))
    rng = np.random.default_rng(chunk)
    n = 2 * chunk + 70
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    want = plain.forward(pcfg, w, base).numpy()
    for run in (run_whole, lambda e, t: run_tail_by_one(e, t, tail=40)):
        ref = run(eng, base)
        assert close(ref, want, "float32")
        for i in (n - 1, n - 17):
            inside = i - i % chunk
            for j, seen in ((inside, True), (inside - 1, False)):
                other = list(base)
                other[j] = (other[j] + 1 + j % 5) % cfg["vocab"]
                got = run(eng, other)
                moved = float(np.abs(got[i] - ref[i]).max())
                # outside the chunk nothing of position i's arithmetic changes at all
                assert (moved > 1e-6) if seen else (moved == 0.0), (chunk, i, j, moved)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_chunk_edge_in_the_fast_kernels(tmp_path_factory, dtype):
    """Heads of 64 and chunks of 100 (the tensor-core kernels in bfloat16): the same dependence,
    with the query projection raised so that single keys carry the rows."""
    def sharpen(tensors):
        tensors["l0.mix.q"] = (tensors["l0.mix.q"].float() * 3.0).to(torch.bfloat16)
    chunk = 100
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention",
                                            tiny._att(4, 2, 64, 64, chunk, 0.2), edit=sharpen,
                                            dtype=dtype)
    rng = np.random.default_rng(4)
    n = 300
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    want = plain.forward(pcfg, w, base).numpy()
    # (far from a chunk's start the slope leaves its first key little weight: the positions
    # looked at are a few keys into the third chunk, in a prompt, decoded, and in a portion that
    # starts two keys into the chunk)
    for run in (run_whole, lambda e, t: run_tail_by_one(e, t, tail=95),
                lambda e, t: run_chunks(e, t, [130, 2, 70])):
        ref = run(eng, base)
        assert close(ref, want, dtype)
        for i in (203, 207, 212):
            first = i - i % chunk
            for j, seen in ((first, True), (first - 1, False)):
                # of a few other tokens at j, the one that moves the plain logits most (a
                # change below bfloat16's resolution would show nothing)
                best, other = -1.0, None
                for c in range(1, 8):
                    cand = list(base)
                    cand[j] = (base[j] + 11 * c) % cfg["vocab"]
                    by = float(np.abs(plain.forward(pcfg, w, cand).numpy()[i] - want[i]).max()) \
                        if seen else 0.0
                    if by > best:
                        best, other = by, cand
                moved = float(np.abs(run(eng, other)[i] - ref[i]).max())
                if seen:
                    assert best > 0.01 * np.abs(want).max() and moved > 0.2 * best, \
                        (dtype, i, j, moved, best)
                else:
                    assert moved == 0.0, (dtype, i, j, moved)


def test_a_loud_sink_and_shut_gates(tmp_path_factory):
    """Sinks of several units either way and gates far from one half: leaving the sink out,
    gating with the wrong head's or channel's number, or mixing the two gates up would move the
    logits by far more than the bound."""
    def edit(tensors):
        if "l0.mix.sink" in tensors:
            tensors["l0.mix.sink"] = torch.tensor([5.0, -4.0, 3.0, 6.0]).to(torch.bfloat16)
        tensors["l0.mix.g"] = (tensors["l0.mix.g"].float() * 4.0).to(torch.bfloat16)
    for kind in ("latent_attention_2", "latent_attention"):
        for dtype in ("float32", "bfloat16"):
            eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, kind, None, edit=edit,
                                                    dtype=dtype)
            toks = np.random.default_rng(5).integers(0, cfg["vocab"], size=120).tolist()
            want = plain.forward(pcfg, w, toks).numpy()
            assert close(run_whole(eng, toks), want, dtype)
            assert close(run_tail_by_one(eng, toks, tail=30), want, dtype)
            if kind == "latent_attention_2":
                w2 = dict(w)
                w2["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -30.0)
                assert rel_err(plain.forward(pcfg, w2, toks).numpy(), want) > 0.02


@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2"])
def test_a_far_key_among_hundreds(tmp_path_factory, kind):
    """Latent attention sees every earlier key; with sharpened queries most of a row's weight
    lies on one key, often far back and beyond block borders, the first tokens included.  The
    rotated part alone is sharpened too: a wrong angle or pairing would move the weight."""
    def sharpen(tensors):
        tensors["l0.mix.uq"] = (tensors["l0.mix.uq"].float() * 6.0).to(torch.bfloat16)
    for mixer in (tiny._lat(4, 16, 8, 16, 32, 24, 0.2), tiny._lat(2, 16, 32, 24, 64, 40, 0.2, 50.0)):
        eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, kind, mixer, edit=sharpen)
        toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=420).tolist()
        want = plain.forward(pcfg, w, toks).numpy()
        assert close(run_whole(eng, toks), want, "float32")
        assert close(run_tail_by_one(eng, toks, tail=50), want, "float32")
        # the first token is among the keys that matter: another first token, other logits
        other = [(toks[0] + 5) % cfg["vocab"]] + toks[1:]
        want2 = plain.forward(pcfg, w, other).numpy()
        assert np.abs(want2[3] - want[3]).max() > 1e-3 * np.abs(want).max()
        assert close(run_tail_by_one(eng, other, tail=417), want2, "float32")


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """``load(...).generate(...)``: batching, the decode graph and the run-ahead of the host,
    against re-running the plain model on the growing sequence."""
    import cretif_b200
    eng = cretif_b200.load(folders[name], dtype="float32", max_tokens=2048)
    pcfg, w = plain.read_model_folder(folders[name])
    prompts = [tiny.tokens(name, n, 40) for n in (3, 11, 30)]
    for use_graph in (True, False):
        got = eng.generate(prompts, max_tokens=12, stop_ids=[], use_graph=use_graph)
        for p, r in zip(prompts, got):
            seq = list(p)
            for tok in r.tokens:        # every token is the plain model's best, or tied with it
                row = plain.forward(pcfg, w, seq)[-1].numpy()
                assert row.max() - row[tok] <= 1e-4 * np.abs(row).max(), (name, use_graph)
                seq.append(tok)
            assert len(r.tokens) == 12
    eng.cache.check()
    assert eng.cache.stats()["slots_live"] == 0


def test_the_replay_program_runs_a_mipurax_folder(folders, tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = tiny.tokens("A", 30, 50)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:20], "want": [0, 19]},
                                     {"id": "y", "tokens": toks[:7], "want": [6]}], "end": ["y"]},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[20:21], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[21:22], "want": []}],
              "end": ["x"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model",
                        folders["A"], "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == \
        ["done 0", "done 1", "done 2"]
    cfg, w = plain.read_model_folder(folders["A"])
    want = plain.forward(cfg, w, toks).numpy()
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    assert not (out / "2.f32").exists()
    assert rel_err(got0, want[[0, 19, 6]]) <= 1e-4 and rel_err(got1, want[[20]]) <= 1e-4


def test_the_command_line_writes_and_runs_a_mipurax_folder(tmp_path):
    """``python -m cretif_b200``: a folder with random weights from a config.json, then greedy
    generation from token ids, the same tokens as the entry point gives."""
    import subprocess
    import sys
    import cretif_b200
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(tiny.M_A))
    folder = str(tmp_path / "model")
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "cretif_b200", folder, "5,6,7,8", "6", "--dtype",
                        "float32", "--random-weights", "21", "--config", str(cfg_file)],
                       capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "model: Mipurax" in r.stdout
    line = [l for l in r.stdout.splitlines() if l.startswith("generated ids:")][0]
    got = json.loads(line[len("generated ids:"):line.index("(")].strip())
    eng = cretif_b200.load(folder, dtype="float32", max_tokens=512)
    want = eng.generate([[5, 6, 7, 8]], max_tokens=6, stop_ids=[])[0].tokens
    assert got == want and len(got) == 6
