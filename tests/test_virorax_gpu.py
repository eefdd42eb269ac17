"""Virorax through the engine against the plain implementation (``plain_virorax``): every
mechanism alone, every way of cutting requests into steps, windows' edges, far memory, reused
slots, greedy generation through the library's own entry point."""
import json
import os

import numpy as np
import pytest
import torch

import plain_virorax as plain
import virorax_tiny as tiny
from replay_cuts import (rel_err, run_batch, run_chunks, run_schedule, run_tail_by_one,
                         run_whole)

pytestmark = pytest.mark.gpu

# Relative to the largest plain logit.  The float32 runs are the sharp ones; bfloat16 rounds
# activations, keys and values to eight bits several times a layer, so its bound is on the mean
# over the positions with a loose one on the worst.  Fewer than four positions give no mean to
# speak of: a lone token's retention read-out is (q.k) v divided by its own root mean square,
# which turns on the sign and size of one dot product when that is near zero.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
BF16_WORST = 0.5


def close(got, want, dtype):
    if dtype == "float32":
        return rel_err(got, want) <= TOL[dtype]
    want = np.asarray(want, dtype=np.float64)
    per_row = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=-1) / np.abs(want).max()
    if len(per_row) < 4:
        return per_row.max() <= BF16_WORST
    return per_row.mean() <= TOL[dtype] and per_row.max() <= BF16_WORST


LENGTHS = {"A": [1, 2, 3, 10, 23, 75, 140], "B": [1, 5, 64, 65, 131, 200], "C": [1, 2, 9, 40],
           "D": [1, 4, 31, 70, 100], "E": [1, 2, 33, 129, 260]}


def _write(tmp_path_factory, name, cfg, seed, edit=None):
    """A model folder for ``cfg`` with seeded random weights; ``edit(tensors)`` may change
    tensors before they are written."""
    from cretif_b200.config import build_virorax_spec, virorax_config_from_dict
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights.loader import random_weights, write_model_folder
    d = str(tmp_path_factory.mktemp(f"virorax_{name}"))
    names, _ = manifest(build_virorax_spec(virorax_config_from_dict(cfg)))
    tensors = random_weights(names, seed, torch.bfloat16)
    # wider projections than the default draw: scores, gates and sinks that are not all alike
    for k in tensors:
        if k.endswith((".q", ".k", ".v", ".g", ".up", ".down", ".o")) or k in ("embed", "pos"):
            tensors[k] = (tensors[k].float() * 4.0).to(torch.bfloat16)
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

    def get(name, dtype, max_tokens=2048, folder=None):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(folder or folders[name], dtype=dtype, max_tokens=max_tokens)
        return made[key]
    return get


@pytest.fixture(scope="module")
def plain_logits(folders):
    models, memo = {}, {}

    def get(name, toks, folder=None):
        key = (name, tuple(toks))
        if key not in memo:
            if name not in models:
                models[name] = plain.read_model_folder(folder or folders[name])
            cfg, w = models[name]
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        return memo[key]
    return get


# ------------------------------------------------------------------ registry and loading
def test_the_configuration_picks_the_model_and_its_parts(folders):
    from cretif_b200.config import load_config
    from cretif_b200.engine import Engine
    arch, cfg, spec = load_config(folders["A"])
    assert arch.name == "Virorax" and spec.vocab_size == 96 and spec.hidden_size == 64
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    eng = Engine(folders["A"], dtype="float32", max_tokens=256)
    groups = eng.cache.stats()["groups"]
    # the three runs of the repeated attention layer share a group, three caches in it
    assert sorted((g["head_dim"], g["layers"], g["window"]) for g in groups) == \
        [(16, 1, 21), (16, 3, 9)]
    assert eng.cache.stats()["state_bytes"] > 0
    assert eng.cache.max_len <= 512                       # the learned positions bound it


# ------------------------------------------------------------------ kernels of the mechanisms
def test_learned_positions_join_the_embedding():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    for dt in (torch.float32, torch.bfloat16):
        table = torch.randn(50, 72, generator=g).to(dt)
        pos = torch.randn(33, 72, generator=g).to(dt)
        ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32)
        at = torch.tensor([32, 0, 5, 5], dtype=torch.int32)
        out = torch.empty(4, 72, device="cuda")
        fault = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.embed_rows(table.cuda(), ids.cuda(), out, fault, positions=pos.cuda(),
                       tok_pos=at.cuda())
        want = table[ids.long()].float() + pos[at.long()].float()
        assert torch.equal(out.cpu(), want) and int(fault.item()) == 0
        ops.embed_rows(table.cuda(), ids.cuda(), out, fault, positions=pos.cuda(),
                       tok_pos=torch.tensor([32, 33, 0, 0], dtype=torch.int32).cuda())
        assert int(fault.item()) == 1 and bool((out[1] == 0).all())    # beyond the table


def test_small_row_kernels():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    x = torch.randn(37, 50, generator=g) * 3
    for kind, f in (("relu2", plain.relu_squared), ("silu", plain.silu),
                    ("gelu_tanh", lambda z: 0.5 * z * (1 + torch.tanh(
                        (2 / torch.pi) ** 0.5 * (z + 0.044715 * z ** 3))))):
        out = torch.empty(37, 50, device="cuda")
        ops.activation(x.cuda(), out, kind)
        assert (out.cpu().double() - f(x.double())).abs().max() < 1e-5
        out = torch.empty(37, 50, device="cuda", dtype=torch.bfloat16)
        ops.activation(x.cuda(), out, kind)
        want = f(x.double())
        assert ((out.cpu().double() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-3).all()
    z = (torch.randn(9, 33, generator=g) * 20).cuda()
    want = plain.soft_cap(z.cpu().double(), 7.5)
    ops.softcap(z, 7.5)
    assert (z.cpu().double() - want).abs().max() < 1e-5 and float(z.abs().max()) <= 7.5
    h = torch.randn(20, 48, generator=g)
    y = torch.randn(20, 48, generator=g)
    for yy in (y, y.bfloat16()):
        got = h.cuda()
        ops.axpy_rows(got, yy.cuda(), 0.3)
        assert (got.cpu().double() - (h.double() + 0.3 * yy.double())).abs().max() < 1e-6
    o = torch.randn(11, 3 * 20, generator=g)
    gate = torch.randn(11, 40, generator=g)
    got = o.cuda()
    ops.gate_heads(got, gate.cuda()[:, 5:8], 3, 20)
    want = (o.double().reshape(11, 3, 20) * torch.sigmoid(gate[:, 5:8].double())[:, :, None])
    assert (got.cpu().double() - want.reshape(11, 60)).abs().max() < 1e-6
    # bfloat16 rows inside a wider buffer: heads of 24 go eight channels a thread, of 20 one
    for vd in (24, 20):
        ob = torch.randn(11, 3 * vd + 8, generator=g).bfloat16()
        buf = ob.cuda()
        ops.gate_heads(buf[:, :3 * vd], gate.cuda()[:, 5:8], 3, vd)
        want = (ob[:, :3 * vd].double().reshape(11, 3, vd)
                * torch.sigmoid(gate[:, 5:8].double())[:, :, None]).reshape(11, 3 * vd)
        assert ((buf[:, :3 * vd].cpu().double() - want).abs() <= 2.0 ** -8 * want.abs()).all()
        assert torch.equal(buf[:, 3 * vd:].cpu(), ob[:, 3 * vd:])


def _cache_for(positions, nkv, hd, dtype, bt=64):
    n_blocks = (positions + bt - 1) // bt + 1
    kc = torch.zeros(n_blocks, nkv, bt, hd, dtype=dtype, device="cuda")
    table = torch.arange(1, n_blocks + 1, dtype=torch.int32, device="cuda").flip(0)[None, :] - 1
    return kc, table.contiguous()


def _gather(cache, table, positions, bt=64):
    t = table[0].cpu()
    return torch.stack([cache[t[p // bt], :, p % bt].cpu() for p in range(positions)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,rot,pairing", [(4, 2, 16, 16, 8, 0), (3, 1, 12, 20, 4, 0),
                                                 (2, 2, 128, 64, 128, 0), (1, 1, 8, 8, 2, 1),
                                                 (2, 1, 72, 130, 0, 0), (1, 1, 300, 40, 100, 0)])
def test_bias_head_norm_rotation_and_cache_write(dtype, H, G, d, e, rot, pairing):
    """The kernel between an attention's projections and its scores, over a sequence fed in
    pieces, against the plain functions."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.position import rotary_table
    g = torch.Generator().manual_seed(3)
    S, base = 90, 300.0
    n_in = (H + G) * d + G * e
    proj = torch.randn(S, n_in + H, generator=g) * 2
    bias = torch.randn(n_in, generator=g)
    wq, wk = torch.randn(d, generator=g), torch.randn(d, generator=g)
    P = proj.double()[:, :n_in] + bias.double()
    q = plain.unit(P[:, :H * d].reshape(S, H, d), 1e-5) * wq.double()
    k = plain.unit(P[:, H * d:(H + G) * d].reshape(S, G, d), 1e-5) * wk.double()
    v = P[:, (H + G) * d:].reshape(S, G, e)
    if rot and not pairing:
        q, k = plain.rotate_front(q, base, rot), plain.rotate_front(k, base, rot)
    elif rot:                       # neighbours are pairs: the same rotation on permuted channels
        perm = list(range(0, rot, 2)) + list(range(1, rot, 2)) + list(range(rot, d))
        inv = [perm.index(i) for i in range(d)]
        q = plain.rotate_front(q[..., perm], base, rot)[..., inv]
        k = plain.rotate_front(k[..., perm], base, rot)[..., inv]
    cos = sin = None
    if rot:
        cos, sin = rotary_table(base, rot, S, torch.device("cuda"))
    kc, table = _cache_for(S, G, d, dtype)
    vc, _ = _cache_for(S, G, e, dtype)
    q_out = torch.zeros(S, H * d + 8, dtype=dtype, device="cuda")
    fault = torch.zeros(1, dtype=torch.int32, device="cuda")
    at = 0
    for n in (1, 2, 30, 1, 56):
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        zeros = torch.zeros(n, dtype=torch.int32, device="cuda")
        ops.headnorm_rope_kv_append(proj[at:at + n].cuda(), bias.cuda(), wq.cuda(), wk.cuda(),
                                    1e-5, cos, sin, pairing, rot, pos, zeros, zeros[:1], H, G, d,
                                    e, q_out[at:at + n], table=table, kc=kc, vc=vc, fault=fault)
        at += n
    assert at == S and int(fault.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (q_out[:, :H * d].cpu().double() - q.reshape(S, H * d)).abs().max() < tol * 4
    assert bool((q_out[:, H * d:] == 0).all())
    assert (_gather(kc, table, S).double() - k).abs().max() < tol * 4
    assert (_gather(vc, table, S).double() - v).abs().max() < tol * 4
    # without weights and bias: rotation and the store alone
    q2 = torch.zeros(S, H * d, dtype=dtype, device="cuda")
    pos = torch.arange(S, dtype=torch.int32, device="cuda")
    ops.headnorm_rope_kv_append(proj.cuda(), None, None, None, 0.0, cos, sin, 0, rot, pos, None,
                                None, H, G, d, e, q2, write_cache=False)
    want = P0 = proj.double()[:, :H * d].reshape(S, H, d)
    if rot:
        want = plain.rotate_front(P0, base, rot)
    assert (q2.cpu().double() - want.reshape(S, H * d)).abs().max() < tol * 8


@pytest.mark.parametrize("H,d,e,rot", [(4, 16, 24, 8), (2, 32, 32, 32), (1, 8, 8, 0), (3, 12, 6, 4),
                                       (2, 128, 64, 64), (1, 72, 130, 2), (1, 300, 40, 20),
                                       (1, 64, 256, 64), (5, 4, 3, 4)])
def test_retention_kernels_in_pieces(H, d, e, rot):
    """Rotation, recurrence, norm and gate over a sequence fed in pieces of 1 to 40 tokens into
    a slot's state, against the recurrence written out token by token."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.position import rotary_table
    g = torch.Generator().manual_seed(5)
    S, base = 97, 1000.0
    proj = torch.randn(S, 2 * H * d + 2 * H * e + 3, generator=g)
    decay = torch.tensor([0.999, 0.9, 0.5, 1.0, 0.97][:H])
    P = proj.double()
    qq = P[:, :H * d].reshape(S, H, d)
    kk = P[:, H * d:2 * H * d].reshape(S, H, d)
    if rot:
        qq, kk = plain.rotate_front(qq, base, rot), plain.rotate_front(kk, base, rot)
    vv = P[:, 2 * H * d:2 * H * d + H * e].reshape(S, H, e)
    o = plain.retention(qq, kk * d ** -0.5, vv, decay.double())
    gate = P[:, 2 * H * d + H * e:2 * H * d + 2 * H * e]
    want = plain.unit(o, 1e-5).reshape(S, H * e) * plain.silu(gate)
    cos = sin = None
    if rot:
        cos, sin = rotary_table(base, rot, S, torch.device("cuda"))
    slots, slot = 3, 2
    state = torch.zeros(slots, H * d * e, device="cuda")
    state[1] = 7.0                                     # a neighbour's state must not be touched
    seq_slot = torch.tensor([slot], dtype=torch.int32, device="cuda")
    got, at = [], 0
    for n in (1, 2, 1, 17, 40, 3, 33):
        n = min(n, S - at)
        rows = proj[at:at + n].cuda().contiguous()
        prep = torch.empty(n, 2 * H * d, device="cuda")
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        ops.retention_prepare(rows, prep, cos, sin, 0, rot, pos, H, d, d ** -0.5)
        o_raw = torch.empty(n, H * e, device="cuda")
        ops.retention_recurrence(prep, rows[:, 2 * H * d:2 * H * d + H * e], decay.cuda(), state,
                                 cu, seq_slot, 1, H, d, e, o_raw)
        out = torch.empty(n, H * e, device="cuda")
        ops.heads_out_norm(o_raw, rows[:, 2 * H * d + H * e:], None, 1e-5, out, H, e)
        assert (o_raw.cpu().double() - o[at:at + n].reshape(n, H * e)).abs().max() \
            <= 1e-4 * max(1.0, float(o.abs().max()))
        got.append(out.cpu())
        at += n
    assert at == S
    got = torch.cat(got).double()
    assert (got - want).abs().max() <= 2e-4 * max(1.0, want.abs().max())
    assert bool((state[1] == 7.0).all()) and bool((state[0] == 0.0).all())
    # a state that is read but not written
    before = state.clone()
    ops.retention_recurrence(prep, rows[:, 2 * H * d:2 * H * d + H * e], decay.cuda(), state, cu,
                             seq_slot, 1, H, d, e, o_raw, write_state=False)
    assert torch.equal(state, before)


@pytest.mark.parametrize("H,d,e", [(2, 128, 128), (3, 32, 64), (1, 64, 16), (5, 16, 48),
                                   (2, 20, 32), (1, 256, 32)])
def test_retention_sixty_four_tokens_at_a_time(H, d, e):
    """The chunked form of the recurrence against the recurrence written out, over sequences of
    unequal length fed in pieces that end before, at and after a chunk's edge, with the state
    carried from piece to piece; the state it leaves equals the token-by-token form's."""
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(11)
    lens = [331, 64, 129]
    decay = torch.tensor([0.999, 0.5, 1.0, 0.97, 0.9][:H])
    seqs = [(torch.randn(n, 2 * H * d, generator=g), torch.randn(n, H * e, generator=g))
            for n in lens]
    want = [plain.retention(p[:, :H * d].double().reshape(-1, H, d),
                            p[:, H * d:].double().reshape(-1, H, d) * d ** -0.5,
                            v.double().reshape(-1, H, e), decay.double()).reshape(-1, H * e)
            for p, v in seqs]
    scale = max(1.0, max(float(w.abs().max()) for w in want))
    slots = torch.tensor([3, 0, 2], dtype=torch.int32, device="cuda")
    states = {}
    for form in ("chunk", "token"):
        state = torch.zeros(5, H * d * e, device="cuda")
        state[1] = 7.0
        at = [0, 0, 0]
        for cuts in ((63, 64, 1), (2, 0, 64), (65, 0, 64), (1, 0, 0), (200, 0, 0)):
            live = [i for i, n in enumerate(cuts) if n]
            prep = torch.cat([seqs[i][0][at[i]:at[i] + cuts[i]] for i in live]).cuda()
            prep[:, H * d:] *= d ** -0.5
            v = torch.cat([seqs[i][1][at[i]:at[i] + cuts[i]] for i in live]).cuda()
            cu = torch.tensor(np.cumsum([0] + [cuts[i] for i in live]), dtype=torch.int32,
                              device="cuda")
            o_raw = torch.full((prep.shape[0], H * e), float("nan"), device="cuda")
            ops.retention_recurrence(prep, v, decay.cuda(), state, cu, slots[live].contiguous(),
                                     len(live), H, d, e, o_raw, form=form)
            row = 0
            for i in live:
                got = o_raw[row:row + cuts[i]].cpu().double()
                ref = want[i][at[i]:at[i] + cuts[i]]
                assert (got - ref).abs().max() <= 2e-5 * scale, (form, cuts, i)
                row += cuts[i]
                at[i] += cuts[i]
        assert at == lens
        assert bool((state[1] == 7.0).all()) and bool((state[4] == 0.0).all())
        states[form] = state
    diff = (states["chunk"] - states["token"]).abs().max()
    assert diff <= 2e-5 * max(1.0, float(states["token"].abs().max()))


def test_the_chunked_form_is_refused_where_it_cannot_run():
    from cretif_b200.csrc import ops
    H, d, e, T = 1, 6, 16, 70
    args = (torch.zeros(T, 2 * H * d, device="cuda"), torch.zeros(T, H * e, device="cuda"),
            torch.ones(H, device="cuda"), torch.zeros(1, H * d * e, device="cuda"),
            torch.tensor([0, T], dtype=torch.int32, device="cuda"),
            torch.zeros(1, dtype=torch.int32, device="cuda"), 1, H, d, e,
            torch.empty(T, H * e, device="cuda"))
    with pytest.raises(ops.KernelError):
        ops.retention_recurrence(*args, form="chunk")
    ops.retention_recurrence(*args, form="auto")          # takes the other form


def test_retention_of_several_sequences_in_one_launch():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(6)
    H, d, e = 3, 16, 20
    lens = [5, 1, 40, 18]
    T = sum(lens)
    prep = torch.randn(T, 2 * H * d, generator=g)
    v = torch.randn(T, H * e, generator=g)
    decay = torch.tensor([0.9, 0.99, 0.8])
    state = torch.zeros(6, H * d * e, device="cuda")
    slots = torch.tensor([4, 0, 5, 2], dtype=torch.int32, device="cuda")
    cu = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device="cuda")
    o_raw = torch.empty(T, H * e, device="cuda")
    ops.retention_recurrence(prep.cuda(), v.cuda(), decay.cuda(), state, cu, slots, 4, H, d, e,
                             o_raw)
    at = 0
    for n in lens:
        q = prep[at:at + n, :H * d].double().reshape(n, H, d)
        k = prep[at:at + n, H * d:].double().reshape(n, H, d)
        want = plain.retention(q, k, v[at:at + n].double().reshape(n, H, e), decay.double())
        assert (o_raw[at:at + n].cpu().double() - want.reshape(n, H * e)).abs().max() < 1e-4
        at += n
    assert bool((state[1] == 0).all()) and bool((state[3] == 0).all())


@pytest.mark.parametrize("H,G,d,window", [(6, 2, 64, 100), (4, 1, 128, 40), (2, 2, 32, 129)])
def test_fast_attention_kernels_with_a_sink_and_a_gate(H, G, d, window):
    """The bfloat16 attention kernels the engine picks (prompt, portion, single tokens) with a
    learned sink, against the plain softmax on the same rounded inputs; a key at each window's
    edge stands out."""
    from cretif_b200.parts.attention import run_attention
    from cretif_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(7)
    S = 333
    q = torch.randn(S, H, d, generator=g)
    k = torch.randn(S, G, d, generator=g)
    for i in range(S):
        k[max(0, i - window + 1), :, 0] += 3.0
        q[i, :, 0] += 2.0
    q, k = q.bfloat16(), k.bfloat16()
    v = torch.randn(S, G, d, generator=g).bfloat16()
    sink = torch.randn(H, generator=g) * 2
    scale = 0.7 / d ** 0.5
    vis = plain.window_mask(S, window)
    want = torch.zeros(S, H, d, dtype=torch.float64)
    for h in range(H):
        w = plain.softmax_with_sink((q[:, h].double() @ k[:, h // (H // G)].double().T) * scale,
                                    vis, sink[h].double())
        want[:, h] = w @ v[:, h // (H // G)].double()
    want = want.reshape(S, H * d)
    kc, table = _cache_for(S, G, d, torch.bfloat16)
    vc = torch.zeros_like(kc)
    t = table[0].cpu()
    for p in range(S):
        kc[t[p // 64], :, p % 64] = k[p].cuda()
        vc[t[p // 64], :, p % 64] = v[p].cuda()

    class KV:
        pass
    kv = KV()
    kv.k, kv.v, kv.table, kv.block_tokens, kv.window = kc, vc, table, 64, window
    dev = torch.device("cuda")
    i32 = dict(dtype=torch.int32, device=dev)
    fault = torch.zeros(1, **i32)

    def ctx(T, first, decode):
        return StepContext(T=T, B=1, tok_ids=torch.zeros(T, **i32),
                           tok_pos=torch.arange(first, first + T, **i32),
                           tok_seq=torch.zeros(T, **i32), seq_slot=torch.zeros(1, **i32),
                           seq_start=torch.tensor([first], **i32),
                           cu_seqlens=torch.tensor([0, T], **i32), is_decode=decode, max_new=T,
                           max_context=512 if decode else first + T, fault=fault,
                           dtype=torch.bfloat16, device=dev)
    for first, T, decode in ((0, S, False), (200, S - 200, False), (S - 1, 1, True),
                             (150, 1, True)):
        out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=dev)
        run_attention(q[first:first + T].reshape(T, H * d).cuda(), out, ctx(T, first, decode), kv,
                      H, G, d, scale, window, torch.bfloat16, sink.cuda())
        err = (out.cpu().double() - want[first:first + T]).abs().max()
        assert err <= 2e-2 * want.abs().max(), (first, T, decode, float(err))
    assert int(fault.item()) == 0


# ------------------------------------------------------------------ each mixer alone in a model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "retention"])
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


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_the_stream_after_every_layer_run(engines, folders, name):
    """The residual stream after each run of each layer, the repeated span's further passes
    and the input added before them included."""
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
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
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


@pytest.mark.parametrize("name", ["A", "E"])
def test_few_token_steps_with_and_without_the_fused_kernels(folders, plain_logits, name):
    """bfloat16 steps of a few tokens norm the rows inside the input product, apply the
    feed-forward's activation and the residual multiplier in the products' epilogues; with the
    few-token kernels switched off the same steps take the separate kernels.  Both ways give the
    plain implementation's logits, and each other's up to the order of summation."""
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
    assert rel_err(got[True][0], got[False][0]) < 2e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_portions_of_a_prompt(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    n = LENGTHS[name][-1]
    toks = tiny.tokens(name, n, 3)
    want = plain_logits(name, toks)
    for cuts in ([2, 2, 2, 2], [63, 2, 64], [1, 70, 1, 2], [5] * 12, [n - 2, 2]):
        assert close(run_chunks(eng, toks, cuts), want, dtype), (name, cuts)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_unequal_batches_against_each_alone_and_reused_slots(engines, plain_logits, name, dtype):
    """Batches of unequal requests on a cache too small for two batches: the second and third
    rounds get slots, blocks and states that were used before."""
    eng = engines(name, dtype, max_tokens=960 if name == "E" else 640)
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
def test_long_decoding_past_every_window(engines, plain_logits, dtype):
    """A short prompt and then 230 single tokens: both windows of B (70 and 130 keys) pass over
    decoded tokens and over block borders, and window blocks are given back on the way."""
    eng = engines("B", dtype)
    toks = tiny.tokens("B", 240, 5)
    got = run_tail_by_one(eng, toks, tail=230)
    assert close(got, plain_logits("B", toks), dtype)
    eng.cache.check()


# ------------------------------------------------------------------ what a position may depend on
def _one_layer_engine(tmp_path_factory, kind, window, edit=None, dtype="float32", mixer=None):
    from cretif_b200.engine import Engine
    cfg = tiny.one_layer(kind, window, mixer=mixer)
    d = _write(tmp_path_factory, f"edge_{kind}_{window}", cfg, seed=13, edit=edit)
    return Engine(d, dtype=dtype, max_tokens=2048), plain.read_model_folder(d), cfg


@pytest.mark.parametrize("window", [1, 7, 64, 65, 129])
def test_a_window_ends_where_it_should(tmp_path_factory, window):
    """One attention layer alone: the logits at position i depend on the tokens i-window+1 .. i
    and on nothing else.  Changing the token just inside the window changes them, changing the
    token just outside does not, for a position inside a prompt and for a decoded one."""
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention", window)
    rng = np.random.default_rng(window)
    n = window + 70
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    want = plain.forward(pcfg, w, base).numpy()
    for run in (run_whole, lambda e, t: run_tail_by_one(e, t, tail=40)):
        ref = run(eng, base)
        assert close(ref, want, "float32")
        for i in (n - 1, n - 17):
            inside, outside = i - window + 1, i - window
            for j, seen in ((inside, True), (outside, False)):
                other = list(base)
                other[j] = (other[j] + 1 + j % 5) % cfg["vocab"]
                got = run(eng, other)
                moved = float(np.abs(got[i] - ref[i]).max())
                # outside the window nothing of position i's arithmetic changes at all
                assert (moved > 1e-6) if seen else (moved == 0.0), (window, i, j, moved)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_window_edge_in_the_fast_kernels(tmp_path_factory, dtype):
    """Heads of 64 and a window of 100 (the tensor-core kernels in bfloat16): the same
    dependence, with the query norm's weight raised so that single keys carry the rows."""
    def sharpen(tensors):
        tensors["l0.mix.q.norm"] = (tensors["l0.mix.q.norm"].float() * 5.0).to(torch.bfloat16)
    window = 100
    eng, (pcfg, w), cfg = _one_layer_engine(
        tmp_path_factory, "attention", window, edit=sharpen, dtype=dtype,
        mixer={"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.2,
               "mask": {"size": window}, "rot": {"base": 5000.0, "dims": 32}})
    rng = np.random.default_rng(4)
    n = 300
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    want = plain.forward(pcfg, w, base).numpy()
    for run in (run_whole, lambda e, t: run_tail_by_one(e, t, tail=40),
                lambda e, t: run_chunks(e, t, [130, 2, 70])):
        ref = run(eng, base)
        assert close(ref, want, dtype)
        for i in (n - 1, n - 30):
            for j, seen in ((i - window + 1, True), (i - window, False)):
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
                    assert best > 0.02 * np.abs(want).max() and moved > 0.2 * best, \
                        (dtype, i, j, moved, best)
                else:
                    assert moved == 0.0, (dtype, i, j, moved)


def test_a_loud_sink_and_a_shut_gate(tmp_path_factory):
    """Sinks of several units either way and gates far from one half: leaving the sink out, or
    gating with the wrong head's number, would move the logits by far more than the bound."""
    def edit(tensors):
        tensors["l0.mix.sink"] = torch.tensor([4.0, -4.0, 2.0, 0.5]).to(torch.bfloat16)
        tensors["l0.mix.g"] = (tensors["l0.mix.g"].float() * 4.0).to(torch.bfloat16)
    for dtype in ("float32", "bfloat16"):
        eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention", 40, edit=edit,
                                                dtype=dtype)
        toks = np.random.default_rng(5).integers(0, cfg["vocab"], size=120).tolist()
        want = plain.forward(pcfg, w, toks).numpy()
        assert close(run_whole(eng, toks), want, dtype)
        assert close(run_tail_by_one(eng, toks, tail=30), want, dtype)
        w2 = dict(w)
        w2["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -30.0)
        assert rel_err(plain.forward(pcfg, w2, toks).numpy(), want) > 0.05


def test_memory_of_a_token_far_back(tmp_path_factory):
    """A retention layer alone whose decays are slow: the first token still shows in the logits
    hundreds of tokens later, across prompt portions and single tokens, and the engine carries
    it as the recurrence written out does."""
    eng, (pcfg, w), cfg = _one_layer_engine(
        tmp_path_factory, "retention", 1,
        mixer={"heads": 2, "dim": 64, "vdim": 8, "decay": [0.9995, 1.0],
               "rot": {"base": 100000.0, "dims": 32}})
    rng = np.random.default_rng(8)
    n = 300
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    other = [(base[0] + 3) % cfg["vocab"]] + base[1:]
    want, want_other = (plain.forward(pcfg, w, t).numpy() for t in (base, other))
    assert np.abs(want[-1] - want_other[-1]).max() > 1e-3 * np.abs(want).max()
    for toks, ref in ((base, want), (other, want_other)):
        assert close(run_whole(eng, toks), ref, "float32")
        assert close(run_chunks(eng, toks, [3, 2, 150, 1, 1, 100]), ref, "float32")
        assert close(run_tail_by_one(eng, toks, tail=60), ref, "float32")


def test_a_far_key_among_hundreds(tmp_path_factory):
    """Attention with a window of 300 whose queries are sharpened: most of a row's weight lies
    on one key, often far back and beyond block borders."""
    def sharpen(tensors):
        tensors["l0.mix.q.norm"] = (tensors["l0.mix.q.norm"].float() * 8.0).to(torch.bfloat16)
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention", 300, edit=sharpen)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=420).tolist()
    want = plain.forward(pcfg, w, toks).numpy()
    assert close(run_whole(eng, toks), want, "float32")
    assert close(run_tail_by_one(eng, toks, tail=50), want, "float32")


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """``load(...).generate(...)``: batching, the decode graph (whose warm-up must not advance
    a recurrent state twice) and the run-ahead of the host, against re-running the plain model
    on the growing sequence."""
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


def test_the_replay_program_runs_a_virorax_folder(folders, tmp_path):
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


def test_the_command_line_writes_and_runs_a_virorax_folder(tmp_path):
    """``python -m cretif_b200``: a folder with random weights from a config.json, then greedy
    generation from token ids, the same tokens as the entry point gives."""
    import subprocess
    import sys
    import cretif_b200
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(tiny.V_A))
    folder = str(tmp_path / "model")
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "cretif_b200", folder, "5,6,7,8", "6", "--dtype",
                        "float32", "--random-weights", "21", "--config", str(cfg_file)],
                       capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "model: Virorax" in r.stdout
    line = [l for l in r.stdout.splitlines() if l.startswith("generated ids:")][0]
    got = json.loads(line[len("generated ids:"):line.index("(")].strip())
    eng = cretif_b200.load(folder, dtype="float32", max_tokens=512)
    want = eng.generate([[5, 6, 7, 8]], max_tokens=6, stop_ids=[])[0].tokens
    assert got == want and len(got) == 6
