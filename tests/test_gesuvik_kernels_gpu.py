"""The kernels of the Gesuvik mechanisms, each alone against the plain functions, on inputs
made so that a fault shows: a token far back that only the slowest retention head still
holds, states carried over pieces of every size and over runs side by side, with and without
a rotation; keys that stand out just inside and just outside a window over a cached latent, in
a prompt and decoded, with the blocks behind the window poisoned, a sink and a gate a head;
pairs of neighbours against pairs of halves; a router whose correction changes the choice and
whose identity experts are chosen."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_gesuvik as plain
from semantic_aware_adaptive_kv_cache_precision_b200 import ops
from semantic_aware_adaptive_kv_cache_precision_b200.config import RotarySpec
from semantic_aware_adaptive_kv_cache_precision_b200.ops import mixture
from semantic_aware_adaptive_kv_cache_precision_b200.parts import RotaryHalf, RotaryInterleaved
from test_venanex_kernels_gpu import DEV, TYPES, Cache, close, dev, i32, rounded, step_for

pytestmark = pytest.mark.gpu


def scan_step(lengths, slots, starts):
    """What the recurrences read of a step: where each sequence's tokens start in the step,
    its slot, and every token's position in its sequence."""
    cu = np.concatenate([[0], np.cumsum(lengths)])
    positions = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)])
    return SimpleNamespace(cu_seqlens=i32(cu), slots=i32(slots), sequences=len(lengths),
                           token_seq=i32(np.repeat(np.arange(len(lengths)), lengths)),
                           positions=i32(positions), tokens=int(cu[-1]),
                           max_new=int(max(lengths)), is_decode=all(n == 1 for n in lengths))


def table_of(turn, dim, positions=512):
    part = RotaryHalf(RotarySpec(dim, turn["dims"], turn["base"], positions), "", "float32")
    part.prepare(DEV, positions)
    return part.cos, part.sin


# -- retention -------------------------------------------------------------------------------------

@pytest.mark.parametrize("heads,dim,vdim,decay,turn", [
    (3, 16, 24, (0.5, 0.9, 0.9995), {"base": 1000.0, "dims": 8}),
    (2, 24, 8, (1.0, 0.7), {"base": 50.0, "dims": 24}),
    (5, 12, 20, (1.0, 0.3, 0.8, 0.99, 0.6), None),
    (2, 192, 64, (0.98, 0.999), {"base": 10000.0, "dims": 64}),
    (4, 64, 128, (0.9, 0.95, 0.99, 0.999), {"base": 300.0, "dims": 32}),
    (1, 2, 1, (0.75,), {"base": 10.0, "dims": 2})])
def test_retention_over_pieces_with_a_token_far_back(heads, dim, vdim, decay, turn):
    """The slowest head's key at token 1 is far larger than any later one, and the last query
    points at it (in the numbers the rotation leaves alone, where it leaves any): what that
    head gives at the end is mostly that token's value, faded 398 times."""
    rng = np.random.default_rng(dim + vdim)
    lengths = (400, 3, 70)
    eps = 1e-5
    qk, vc = heads * dim, heads * vdim
    slow = int(np.argmax(decay))
    rot = turn["dims"] if turn else 0
    cos, sin = table_of(turn, dim) if turn else (None, None)
    seqs = []
    for n in lengths:
        proj = rng.standard_normal((n, 7 + 2 * qk + 2 * vc))
        if n > 100 and rot < dim:
            proj[1, 7 + qk + slow * dim + rot:7 + qk + (slow + 1) * dim] = 20.0
            proj[-1, 7 + slow * dim + rot:7 + (slow + 1) * dim] = 6.0
        proj = dev(proj).cpu().numpy().astype(np.float64)
        q, k, v = (proj[:, lo:lo + c].reshape(n, heads, -1)
                   for lo, c in ((7, qk), (7 + qk, qk), (7 + 2 * qk, vc)))
        if turn:
            q, k = plain.turn_halves(q, np.arange(n), turn), plain.turn_halves(k, np.arange(n), turn)
        k = k * dim ** -0.5
        o = np.empty((n, heads, vdim))
        for h in range(heads):
            S = np.zeros((dim, vdim))
            for i in range(n):
                S = decay[h] * S + np.outer(k[i, h], v[i, h])
                o[i, h] = S.T @ q[i, h]
        if n > 100 and rot < dim and decay[slow] > 0.999:
            far = decay[slow] ** (n - 2) * (k[1, slow] @ q[-1, slow]) * v[1, slow]
            assert np.abs(far).max() > 0.5 * np.abs(o[-1, slow]).max()
        gate = proj[:, 7 + 2 * qk + vc:]
        normed = plain.rms_norm(o, None, eps).reshape(n, vc) * plain.silu(gate)
        seqs.append((proj, o.reshape(n, vc), normed))
    less_one = dev(np.asarray(decay, dtype=np.float64) - 1.0)
    state = torch.full((5, heads, vdim, dim), -2.0, device=DEV)
    for cuts, run in (((400, 3, 70), 0), ((1, 1, 1), 0), ((2, 2, 2), 0), ((63, 3, 17), 0),
                      ((399, 1, 70), 0), ((400, 3, 70), 64), ((400, 3, 70), 16), ((130, 3, 33), 32),
                      ((399, 1, 70), 7)):
        slots = [2, 4, 0]
        state[slots] = 0.0
        at = [0] * 3
        raw, rows = [[] for _ in lengths], [[] for _ in lengths]
        while any(a < n for a, n in zip(at, lengths)):
            live = [i for i in range(3) if at[i] < lengths[i]]
            take = [min(cuts[i], lengths[i] - at[i]) for i in live]
            step = scan_step(take, [slots[i] for i in live], [at[i] for i in live])
            proj = dev(np.concatenate([seqs[i][0][at[i]:at[i] + t] for i, t in zip(live, take)]))
            y = ops.decay_attention(proj, 7, 7 + qk, 7 + 2 * qk, heads, dim, vdim, less_one, state,
                                    step, run=run, activation=False, cos=cos, sin=sin,
                                    key_scale=dim ** -0.5)
            out = ops.norm_gate(y, None, proj[:, 7 + 2 * qk + vc:], eps, 1.0, torch.float32,
                                group=vdim, gate_silu=True)
            for i, t, lo in zip(live, take, np.cumsum([0] + take)):
                raw[i].append(y[lo:lo + t])
                rows[i].append(out[lo:lo + t])
                at[i] += t
        for i in range(3):
            close(torch.cat(raw[i]), seqs[i][1], torch.float32,
                  f"cuts {cuts}, runs of {run}, sequence {i}")
            close(torch.cat(rows[i]), seqs[i][2], torch.float32, f"cuts {cuts}, normed {i}")
    before = state.clone()
    ops.decay_attention(dev(seqs[1][0]), 7, 7 + qk, 7 + 2 * qk, heads, dim, vdim, less_one, state,
                        scan_step([3], [4], [0]), keep_state=False, activation=False, cos=cos,
                        sin=sin)
    assert torch.equal(state, before)


@pytest.mark.parametrize("width,group", [(24, 24), (24, 8), (100, 20), (640, 128), (7, 1), (96, 3)])
def test_norm_a_head_with_and_without_weight_and_either_gate(width, group):
    rng = np.random.default_rng(width + group)
    n, eps = 9, 1e-6
    y = dev(rng.standard_normal((n, width)) * 5.0)
    gate = dev(rng.standard_normal((n, width + 3)))[:, 3:]
    w = rounded(1 + 0.2 * rng.standard_normal(width), torch.bfloat16)
    y64, g64 = y.cpu().numpy().astype(np.float64), gate.cpu().numpy().astype(np.float64)
    normed = plain.rms_norm(y64.reshape(n, -1, group), None, eps).reshape(n, width)
    for weight, silu, out_dtype in ((None, True, torch.float32), (w, False, torch.float32),
                                    (w, True, torch.bfloat16), (None, False, torch.bfloat16)):
        want = normed * (1.0 if weight is None else weight) \
            * (plain.silu(g64) if silu else plain.sigmoid(g64)) * 0.7
        got = ops.norm_gate(y, None if weight is None else dev(weight, torch.bfloat16), gate, eps,
                            0.7, out_dtype, group=group, gate_silu=silu)
        close(got, want, out_dtype, f"weight {weight is not None}, silu {silu}")


# -- pairs of neighbours -----------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot,heads,dim", [(40, 8, 4, 16), (36, 6, 5, 12), (512, 64, 2, 128),
                                                (16, 32, 1, 8), (3, 2, 3, 1)])
def test_latent_rows_and_queries_turned_in_pairs_of_neighbours(dtype, rank, rot, heads, dim):
    T = TYPES[dtype]
    rng = np.random.default_rng(rank)
    turn = {"base": 500.0, "dims": rot}
    part = RotaryInterleaved(RotarySpec(rot, rot, 500.0, 512, kind="rotary_interleaved"), "", dtype)
    part.prepare(DEV, 512)
    assert part.interleaved and not RotaryHalf.interleaved
    positions = [0, 1, 63, 64, 200, 511]
    n, eps = len(positions), 1e-5
    down = dev(rng.standard_normal((n, rank + rot)) * 3.0)
    w = rounded(1 + 0.3 * rng.standard_normal(rank), T)
    d64 = down.cpu().numpy().astype(np.float64)
    cache = Cache(1, rank + rot, None, T, seed=6)
    table = cache.table([0], 512)
    step = step_for([0] * n, positions)
    view = SimpleNamespace(keys=cache.keys, block_table=table)
    assert mixture.latent_prepare(down, 0, rank, rot, None, dev(w, T), eps, step, view, part.cos,
                                  part.sin, T, True, True) is None
    rows = table[0].tolist()
    got = torch.stack([cache.keys[rows[p // 64], 0, p % 64] for p in positions])
    want = np.concatenate([plain.rms_norm(d64[:, :rank], w, eps),
                           plain.turn_neighbours(d64[:, None, rank:], positions, turn)[:, 0]], 1)
    close(got, want, T, "the cached rows")
    halves = plain.turn_halves(d64[:, None, rank:], positions, turn)[:, 0]
    if rot > 2:
        assert np.abs(halves - want[:, rank:]).max() > 0.1      # the two pairings differ
    # the queries' rotated part, in place, behind each head's plain part
    q = rounded(rng.standard_normal((n, heads * (dim + rot) + heads)), T)
    x = dev(q, T)
    mixture.rotate_heads(x, dim + rot, dim, heads, rot, step.positions, part.cos, part.sin, True)
    q3 = q[:, :heads * (dim + rot)].reshape(n, heads, dim + rot).copy()
    q3[:, :, dim:] = plain.turn_neighbours(q3[:, :, dim:], positions, turn)
    close(x[:, :heads * (dim + rot)], q3.reshape(n, -1), T, "the queries")
    assert torch.equal(x[:, heads * (dim + rot):], dev(q, T)[:, heads * (dim + rot):])


# -- attention over a cached latent under a window, with a sink and a gate a head ----------------------

def plain_latent_attention(qa, qb, rows, rank, scale, window, sinks, gate):
    n, heads = qa.shape[:2]
    seen = plain.banded(n, window)
    out = np.empty((n, heads, rank))
    for h in range(heads):
        s = (qa[:, h] @ rows[:, :rank].T + qb[:, h] @ rows[:, rank:].T) * scale
        out[:, h] = plain.sink_softmax(s, seen, None if sinks is None else sinks[h]) @ rows[:, :rank]
        if gate is not None:
            out[:, h] *= plain.sigmoid(gate[:, h:h + 1])
    return out.reshape(n, -1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank,rot,window", [(4, 40, 8, 37), (5, 36, 6, 100), (2, 512, 64, 128),
                                                   (1, 16, 32, None), (3, 24, 8, 64), (6, 80, 16, 70),
                                                   (2, 8, 2, 1)])
def test_keys_at_the_window_s_edge_over_a_cached_latent(dtype, heads, rank, rot, window):
    """Three keys stand out: for one asker the oldest key of its window and the one before it,
    and one far back. Each asker's query points at all of them; it must see exactly those that
    its window allows."""
    T = TYPES[dtype]
    rng = np.random.default_rng(rank + rot)
    n, scale = 330, 0.4
    w = window or n
    rows = 0.3 * rng.standard_normal((n, rank + rot))
    qa = 0.3 * rng.standard_normal((n, heads, rank))
    qb = 0.3 * rng.standard_normal((n, heads, rot))
    gate = rng.standard_normal((n, heads))
    sinks = rng.standard_normal(heads)
    asker = 255 + w if 255 + w < n - 1 else 259       # its window starts at a block's first position
    oldest = asker - w + 1
    marked = [p for p in (13, oldest, oldest - 1) if 0 <= p < n]
    for p in marked:
        rows[p] *= 4.0
    for ask in (asker, asker + 1, asker - 1, 13 + w - 1, 13 + w, 14):
        if 0 <= ask < n:
            for h in range(heads):
                qa[ask, h] = sum(rows[p, :rank] for p in marked) * 2.0
                qb[ask, h] = sum(rows[p, rank:] for p in marked) * 2.0
    rows, qa, qb, gate = (rounded(a, T) for a in (rows, qa, qb, gate))
    want = plain_latent_attention(qa, qb, rows, rank, scale, window, sinks, gate)
    assert np.abs(want - plain_latent_attention(qa, qb, rows, rank, scale, window, None, gate)).max() > 0.01
    if window and window < 200:
        assert np.abs(want - plain_latent_attention(qa, qb, rows, rank, scale, None, sinks,
                                                    gate)).max() > 0.05
    cache = Cache(1, rank + rot, None, T, seed=7)
    cache.put(0, rows[:, None, :])
    table = cache.table([0], n)
    gates = dev(np.concatenate([np.zeros((n, 5)), gate], 1), T)[:, 5:]      # rows 5 apart

    def run(cases, tab):
        for lo, hi, across in cases:
            first = across < 0                      # (negative: the heads-first form)
            if dtype == "float32" and first:
                continue
            step = step_for([0] * (hi - lo), range(lo, hi))
            got = ops.cached_attention(dev(qa[lo:hi], T), cache.keys, None, step.positions,
                                       step.token_seq, tab, heads, rank + rot, rank, scale,
                                       q2=dev(qb[lo:hi], T), q_split=rank, window=window,
                                       sink=dev(sinks), head_gate=gates[lo:hi],
                                       key_splits=abs(across), heads_first=first)
            close(got, want[lo:hi], T, f"positions {lo}..{hi}, {across} blocks")

    run([(0, n, 1), (0, 3, 1), (0, 1, -2), (w - 1, min(w + 2, n), 1), (12, 15, 1)], table)
    decoded = table.clone()          # a running sequence no longer holds the blocks behind its window
    if window:
        for b in range(0, oldest // 64):
            cache.keys[table[0, b]] = float("nan")
            decoded[0, b] = -1
    run([(asker, asker + 1, 1), (asker, asker + 2, 1), (asker, asker + 1, -1),
         (asker, asker + 1, -4), (asker + 1, asker + 2, -16)], decoded)


# -- the router: softmax scores, a correction for the choice, identity experts ------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,experts,identity,top,ff", [
    (1, 64, 2, 1, 1, 96), (77, 96, 6, 2, 2, 48), (5, 100, 3, 0, 3, 50), (200, 64, 36, 4, 4, 24),
    (33, 72, 7, 3, 10, 130), (300, 200, 5, 1, 2, 72), (9, 36, 1, 5, 2, 20)])
def test_softmax_router_with_correction_and_identity_experts(dtype, n, width, experts, identity,
                                                             top, ff):
    T = TYPES[dtype]
    rng = np.random.default_rng(n + experts)
    limit = 1.1
    outputs = experts + identity
    h = rounded(rng.standard_normal((n, width)), T)
    t = {"router": rounded(rng.standard_normal((outputs, width)) * 0.3, torch.float32),
         "correction": rounded(rng.standard_normal(outputs) * 0.2, torch.float32)}
    for e in range(experts):
        t[f"e{e}.gate"] = rounded(rng.standard_normal((ff, width)) * 0.2, T)
        t[f"e{e}.up"] = rounded(rng.standard_normal((ff, width)) * 0.2, T)
        t[f"e{e}.down"] = rounded(rng.standard_normal((width, ff)) * 0.2, T)
    mlp = {"router": {"experts": experts, "identity": identity, "top": top},
           "expert": {"ff": ff, "limit": limit}}
    chosen, weights = plain.route(h, t, "", top)
    uncorrected, _ = plain.route(h, {"router": t["router"]}, "", top)
    if n > 30 and top < outputs:
        assert (np.sort(chosen, -1) != np.sort(uncorrected, -1)).any()   # the correction matters
        assert (chosen >= experts).any() or identity == 0                # identity experts occur
    logits = mixture.router_logits(dev(h, T), dev(t["router"]))
    routing = mixture.route(logits, experts, top, identity, True, dev(t["correction"]))
    # a close call may fall either way in 32 bits: rows whose chosen sets differ must be ties
    got_chosen = routing.chosen.cpu().numpy()
    z = h @ t["router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    choice = s / s.sum(-1, keepdims=True) + t["correction"]
    for i in np.flatnonzero((np.sort(got_chosen, -1) != np.sort(chosen, -1)).any(-1)):
        gap = np.abs(np.sort(choice[i, chosen[i]])[0] - np.sort(choice[i, got_chosen[i]])[0])
        assert gap < 1e-6, f"row {i} chose {got_chosen[i]} for {chosen[i]}"
    same = (got_chosen == chosen).all(-1)
    assert same.mean() > 0.95
    assert np.allclose(routing.weights.cpu().numpy()[same], weights[same], rtol=2e-5, atol=1e-7)
    offsets = routing.offsets.cpu().numpy()
    real = got_chosen[got_chosen < experts]
    assert offsets[0] == 0 and offsets[-1] == real.size
    assert np.array_equal(np.diff(offsets), np.bincount(real, minlength=experts))
    rows = mixture.gather_rows(dev(h, T), routing, False)
    slot_of = routing.slot_of.cpu().numpy()
    assert (slot_of[got_chosen >= experts] == -1).all()
    assert sorted(slot_of[got_chosen < experts].tolist()) == list(range(real.size))
    stack = lambda name: dev(np.stack([t[f"e{e}.{name}"] for e in range(experts)]), T)
    act = mixture.grouped_product(rows, routing, stack("gate"), stack("up"), limit, plain.ALPHA)
    products = mixture.grouped_product(act, routing, stack("down"), None)
    shared = rng.standard_normal((n, width))
    out = mixture.combine(products, routing, True, dev(shared), None, dev(h, T))
    want = plain.experts(h, t, "", mlp) + dev(shared).cpu().numpy().astype(np.float64)
    close(out.cpu()[torch.from_numpy(same)], want[same], T, "the routed experts")
    again = mixture.route(logits, experts, top, identity, True, dev(t["correction"]))
    assert torch.equal(again.offsets, routing.offsets)      # the counts were left clean
    # the sigmoid router of the other designs is as it was: chosen by the logits themselves
    old = mixture.route(logits, experts, min(top, experts))
    assert np.array_equal(old.chosen.cpu().numpy(),
                          np.argsort(-logits.cpu().numpy()[:, :experts].astype(np.float64), -1,
                                     kind="stable")[:, :min(top, experts)])
