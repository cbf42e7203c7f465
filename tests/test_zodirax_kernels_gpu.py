"""The kernels of the Zodirax mechanisms, each alone against the plain functions, on inputs
made so that a fault shows: a key that stands out just inside and just outside a window and
the kept first tokens (in a prompt and decoded, at block borders, with freed blocks poisoned),
a sink that outweighs every key, a token far back that a slow channel of the scan and a slow
head of the fading state still hold, states carried over pieces of every size, and slots used
again."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_zodirax as plain
from semantic_aware_adaptive_kv_cache_precision_b200 import ops
from test_venanex_kernels_gpu import DEV, TYPES, Cache, close, dev, i32, rounded, step_for

pytestmark = pytest.mark.gpu


def scan_step(lengths, slots):
    """What the recurrences read of a step: where each sequence's tokens start, and its slot."""
    cu = np.concatenate([[0], np.cumsum(lengths)])
    return SimpleNamespace(cu_seqlens=i32(cu), slots=i32(slots), sequences=len(lengths),
                           token_seq=i32(np.repeat(np.arange(len(lengths)), lengths)),
                           tokens=int(cu[-1]), max_new=int(max(lengths)),
                           is_decode=all(n == 1 for n in lengths))


# -- the norm on a sublayer's output --------------------------------------------------------

@pytest.mark.parametrize("width", [1, 7, 100, 256, 1000, 4100])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_output_norm_completes_the_stream(width, wdtype):
    rng = np.random.default_rng(width)
    n, eps = 5, 1e-5
    x = dev(rng.standard_normal((n, width)) * 3.0)
    y = dev(40.0 * rng.standard_normal((n, width)))
    w1, w2 = (rounded(0.2 * rng.standard_normal(width), wdtype) for _ in range(2))
    x64, y64 = x.cpu().numpy().astype(np.float64), y.cpu().numpy().astype(np.float64)
    want_x = x64 + plain.rms_norm(y64, w1, eps, plus_one=True)
    stream = x.clone()
    low = ops.rms_update(stream, y, add_weight=dev(w1, wdtype), add_offset=1.0,
                         out_dtype=torch.bfloat16, eps=eps)
    assert np.abs(stream.cpu().numpy() - want_x).max() <= 2e-6 * np.abs(want_x).max()
    assert torch.equal(low, stream.to(torch.bfloat16))
    alone = x.clone()
    assert ops.rms_update(alone, y, add_weight=dev(w1, wdtype), add_offset=1.0, eps=eps) is None
    assert torch.equal(alone, stream)
    # the norm of the stream itself (the model's last norm), on chosen rows too
    want = plain.rms_norm(want_x, w2, eps, plus_one=True)
    got = ops.rms_update(stream, out_dtype=torch.float32, out_weight=dev(w2, wdtype),
                         out_offset=1.0, eps=eps)
    assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * max(np.abs(want).max(), 1.0)
    some = ops.rms_update(stream, out_dtype=torch.float32, out_weight=dev(w2, wdtype),
                          out_offset=1.0, eps=eps, rows=i32([3, 0, 3]))
    assert torch.equal(some, got[[3, 0, 3]])
    plain_w = ops.rms_update(stream, out_dtype=torch.float32, out_weight=dev(w2, wdtype), eps=eps)
    want = plain.rms_norm(want_x, w2, eps)
    assert np.abs(plain_w.cpu().numpy() - want).max() <= 2e-5 * max(np.abs(want).max(), 1.0)


# -- norm over the whole projection, partial rotation, the cache write ---------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,turn", [
    (4, 2, 32, 24, {"base": 10000.0, "dims": 16,
                    "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}),
    (6, 2, 20, 12, {"base": 777.0, "dims": 6}), (1, 1, 64, 320, {"base": 300.0, "dims": 64}),
    (3, 1, 24, 36, None)])
def test_whole_projection_norm_rotation_and_cache_write(dtype, heads, kv_heads, dim, vdim, turn):
    from semantic_aware_adaptive_kv_cache_precision_b200.config import BandScaling, RotarySpec
    from semantic_aware_adaptive_kv_cache_precision_b200.parts import RotaryHalf
    T = TYPES[dtype]
    rng = np.random.default_rng(dim)
    n, eps = 150, 1e-5
    qc, kc, vc = heads * dim, kv_heads * dim, kv_heads * vdim
    proj = dev(np.concatenate([rng.standard_normal((n, 5)), 3.0 * rng.standard_normal((n, qc)),
                               0.2 * rng.standard_normal((n, kc)), rng.standard_normal((n, vc))], 1))
    p64 = proj.cpu().numpy().astype(np.float64)
    wq, wk = rounded(1 + 0.3 * rng.standard_normal(qc), T), rounded(1 + 0.3 * rng.standard_normal(kc), T)
    positions = np.arange(n) + 0
    q = plain.rms_norm(p64[:, 5:5 + qc], wq, eps).reshape(n, heads, dim)
    k = plain.rms_norm(p64[:, 5 + qc:5 + qc + kc], wk, eps).reshape(n, kv_heads, dim)
    cos = sin = None
    if turn is not None:
        q, k = plain.rotate_front(q, positions, turn), plain.rotate_front(k, positions, turn)
        sc = turn.get("scaling")
        part = RotaryHalf(RotarySpec(dim, turn["dims"], turn["base"], 256, scaling=None if sc is None
                                     else BandScaling(sc["factor"], sc["original"], sc["low"],
                                                      sc["high"])), "", dtype)
        part.prepare(DEV, 256)
        cos, sin = part.cos, part.sin
    cache = Cache(kv_heads, dim, vdim, T, seed=3)
    table = cache.table([0], n)
    step = step_for([0] * n, positions)
    got = ops.qk_prepare(proj, 5, 5 + qc, 5 + qc + kc, heads, kv_heads, dim, vdim, dev(wq, T),
                         dev(wk, T), eps, cos, sin, step.positions, step.token_seq, table,
                         cache.keys, cache.values, T)
    close(got, q.reshape(n, qc), T, "queries")
    rows = table[0].tolist()
    keys = torch.stack([cache.keys[rows[p // 64], :, p % 64] for p in range(n)])
    values = torch.stack([cache.values[rows[p // 64], :, p % 64] for p in range(n)])
    close(keys, k, T, "keys in the cache")
    close(values, p64[:, 5 + qc + kc:].reshape(n, kv_heads, vdim), T, "values in the cache")


# -- a window that keeps the first tokens, and the sink -------------------------------------------

def plain_window_attention(q, k, v, scale, window, keep, sinks, group):
    n, heads = q.shape[:2]
    seen = plain.visible(n, window if window else n, keep)
    out = np.empty((n, heads, v.shape[-1]))
    for h in range(heads):
        w = plain.sink_softmax(q[:, h] @ k[:, h // group].T * scale, seen,
                               -np.inf if sinks is None else sinks[h])
        out[:, h] = w @ v[:, h // group]
    return out.reshape(n, -1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,keep", [
    (4, 2, 32, 24, 37, 3), (2, 2, 16, 40, 64, 0), (6, 2, 20, 12, 3, 1), (3, 1, 24, 36, 100, 70),
    (4, 1, 128, 128, 128, 5), (1, 1, 64, 320, None, 0), (2, 1, 8, 8, 1, 0)])
def test_keys_at_the_window_s_edge_and_the_kept_first_tokens(dtype, heads, kv_heads, dim, vdim,
                                                            window, keep):
    """Four keys stand out: the last kept token, the first that is not kept, and for one asker
    the oldest key of its window and the one before. Each asker's query points at all four; it
    must see exactly those that its mask allows."""
    T = TYPES[dtype]
    rng = np.random.default_rng(dim + vdim)
    n, scale, out_scale = 330, 0.4, 1.3
    group = heads // kv_heads
    k = 0.3 * rng.standard_normal((n, kv_heads, dim))
    v = rng.standard_normal((n, kv_heads, vdim))
    q = 0.3 * rng.standard_normal((n, heads, dim))
    sinks = rng.standard_normal(heads)
    w = window or n
    # the asker's window starts at a block's first position where the sequence is long enough
    asker = 255 + w if 255 + w < n - 1 else 259
    oldest = asker - w + 1
    marked = [p for p in (keep - 1, keep, oldest, oldest - 1) if 0 <= p < n]
    for p in marked:
        k[p] *= 4.0
    for ask in (asker, asker + 1, max(keep - 1, 0), keep, keep + w - 1, keep + w, 1):
        if ask < n:
            for h in range(heads):
                q[ask, h] = sum(k[p, h // group] for p in marked) * 2.0
    k, v, q = rounded(k, T), rounded(v, T), rounded(q, T)
    want = plain_window_attention(q, k, v, scale, window, keep, sinks, group) * out_scale
    without = plain_window_attention(q, k, v, scale, window, keep, None, group) * out_scale
    assert np.abs(want - without).max() > 0.05      # the sink matters here
    cache = Cache(kv_heads, dim, vdim, T, seed=4)
    cache.put(0, k, v)
    table = cache.table([0], n)

    def run(cases, tab):
        for lo, hi, across in cases:
            first = across < 0                      # (negative: the heads-first form)
            if dtype == "float32" and first:
                continue
            step = step_for([0] * (hi - lo), range(lo, hi))
            got = ops.cached_attention(dev(q[lo:hi], T), cache.keys, cache.values, step.positions,
                                       step.token_seq, tab, heads, dim, vdim, scale, window=window,
                                       keep_first=keep, sink=dev(sinks), out_scale=out_scale,
                                       key_splits=abs(across), heads_first=first)
            close(got, want[lo:hi], T, f"positions {lo}..{hi}, {across} blocks")

    run([(0, n, 1), (0, 3, 1), (0, 1, -2), (keep, keep + 1, -1), (max(keep - 1, 0), keep + 2, 1),
         (max(min(keep + w - 2, n - 3), 0), min(keep + w + 1, n), 1)], table)
    # what a running sequence no longer holds: whole blocks behind the asker's window, but for
    # the kept tokens' blocks
    decoded = table.clone()
    if window:
        for b in range(-(-keep // 64), oldest // 64):
            cache.keys[table[0, b]] = float("nan")
            cache.values[table[0, b]] = float("nan")
            decoded[0, b] = -1
    run([(asker, asker + 1, 1), (asker, asker + 2, 1), (asker, asker + 1, -1),
         (asker, asker + 1, -4), (asker + 1, asker + 2, -16)], decoded)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_whole_prompt_under_the_window_and_two_sequences_of_one_step(dtype):
    """Every query of two prompts of unequal length in one step, blocks in scrambled order; the
    first tokens of each sequence see only what exists; a sink that outweighs every key leaves
    almost nothing."""
    T = TYPES[dtype]
    rng = np.random.default_rng(9)
    heads, kv_heads, dim, vdim, window, keep, scale = 4, 2, 16, 24, 37, 3, 0.5
    lengths = (200, 71)
    cache = Cache(kv_heads, dim, vdim, T, seed=5)
    qs, wants = [], []
    sinks = np.array([0.3, -2.0, 30.0, 0.0])
    for s, n in enumerate(lengths):
        k = rounded(0.5 * rng.standard_normal((n, kv_heads, dim)), T)
        v = rounded(rng.standard_normal((n, kv_heads, vdim)), T)
        q = rounded(0.5 * rng.standard_normal((n, heads, dim)), T)
        cache.put(s, k, v)
        qs.append(q)
        wants.append(plain_window_attention(q, k, v, scale, window, keep, sinks, 2))
    want = np.concatenate(wants)
    assert np.abs(want.reshape(-1, heads, vdim)[:, 2]).max() < 1e-9      # head 2: all to the sink
    table = torch.cat([cache.table([0], 200), cache.table([1], 200)])
    step = step_for([0] * 200 + [1] * 71, list(range(200)) + list(range(71)))
    got = ops.cached_attention(dev(np.concatenate(qs), T), cache.keys, cache.values,
                               step.positions, step.token_seq, table, heads, dim, vdim, scale,
                               window=window, keep_first=keep, sink=dev(sinks))
    close(got, want, T, "two prompts")
    step = step_for([1, 0], [70, 199])              # their last tokens, decoded together
    last = np.stack([qs[1][70], qs[0][199]])
    for across, first in ((1, False), (2, True)):
        if dtype == "float32" and first:
            continue
        got = ops.cached_attention(dev(last, T), cache.keys, cache.values, step.positions,
                                   step.token_seq, table, heads, dim, vdim,
                                   scale, window=window, keep_first=keep, sink=dev(sinks),
                                   key_splits=across, heads_first=first)
        close(got, np.stack([wants[1][70], wants[0][199]]), T, "two last tokens")


# -- the short convolution and its running inputs ------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("channels,taps", [(128, 4), (72, 2), (50, 3), (30, 1), (256, 7)])
def test_convolution_over_pieces_and_slots_used_again(dtype, channels, taps):
    T = TYPES[dtype]
    rng = np.random.default_rng(channels)
    lengths = (41, 3, 1, 17)
    w = rounded(rng.standard_normal((channels, taps)), T)
    b = rounded(rng.standard_normal(channels), T)
    xs = [rng.standard_normal((n, channels + 9)) for n in lengths]          # wider rows
    xs = [dev(x).cpu().numpy().astype(np.float64) for x in xs]
    wants = [plain.silu(plain.causal_conv(x[:, :channels], w, b)) for x in xs]
    state = torch.full((6, taps - 1, channels), 7.0, device=DEV)            # slots left dirty
    for cuts in ((41, 3, 1, 17), (1, 1, 1, 1), (2, 2, 1, 5), (40, 1, 1, 16)):
        slots = [4, 1, 5, 0]
        state[slots] = 0.0                          # what taking a slot does
        at = [0] * 4
        rows = [[] for _ in lengths]
        while any(a < n for a, n in zip(at, lengths)):
            live = [i for i in range(4) if at[i] < lengths[i]]
            take = [min(cuts[i], lengths[i] - at[i]) for i in live]
            step = scan_step(take, [slots[i] for i in live])
            piece = dev(np.concatenate([xs[i][at[i]:at[i] + t] for i, t in zip(live, take)]))
            out = ops.causal_conv(piece, channels, dev(w, T), dev(b, T), state, step, T)
            for i, t, lo in zip(live, take, np.cumsum([0] + take)):
                rows[i].append(out[lo:lo + t])
                at[i] += t
        for i in range(4):
            close(torch.cat(rows[i]), wants[i], T, f"cuts {cuts}, sequence {i}")


# -- step sizes and the selective scan -------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("channels,n_state,rank", [(128, 16, 6), (72, 5, 3), (50, 7, 5), (30, 1, 1),
                                                   (64, 160, 8), (40, 130, 4)])
def test_selective_scan_over_pieces_with_a_token_far_back(dtype, channels, n_state, rank):
    """Channel 0 hardly decays and is fed once, at token 2, far more than anything after it; the
    last token's C reads exactly that state. Pieces down to one token give the same."""
    T = TYPES[dtype]
    rng = np.random.default_rng(channels + n_state)
    lengths = (400, 5, 64)
    a_log = rng.uniform(-3.0, 1.0, (channels, n_state))
    a_log[0] = -9.0                                 # exp(dt A) stays near 1
    a_log, d_skip = rounded(a_log, T), rounded(1 + 0.1 * rng.standard_normal(channels), T)
    w_dt, b_dt = rounded(rng.standard_normal((channels, rank)), T), rounded(rng.uniform(-4, -1, channels), T)
    seqs = []
    for n in lengths:
        x = rng.standard_normal((n, channels))
        low = rng.standard_normal((n, rank + 3 + 2 * n_state))             # columns between
        z = rng.standard_normal((n, channels))
        if n > 100:
            x[2, 0] = 300.0
            low[-1, rank + 3 + n_state:] *= 5.0
        x = rounded(x, T)
        low, z = (dev(a).cpu().numpy().astype(np.float64) for a in (low, z))
        dt = plain.softplus(low[:, :rank] @ w_dt.T + b_dt)
        y = plain.selective_scan(x, dt, -np.exp(a_log), low[:, rank + 3:rank + 3 + n_state],
                                 low[:, rank + 3 + n_state:], d_skip)
        if n > 100:                                 # the far token is felt at the last one
            bare = x.copy()
            bare[2, 0] = 0.0
            other = plain.selective_scan(bare, dt, -np.exp(a_log), low[:, rank + 3:rank + 3 + n_state],
                                         low[:, rank + 3 + n_state:], d_skip)
            assert abs(y[-1, 0] - other[-1, 0]) > 0.05 * np.abs(y[-1]).max()
        seqs.append((x, low, z, dt, y * plain.silu(z)))
    state = torch.full((5, channels, n_state), 3.0, device=DEV)
    # (the second number: tokens a run when a step's part of a sequence is walked in runs)
    for cuts, run in (((400, 5, 64), 0), ((1, 1, 1), 0), ((2, 2, 2), 0), ((63, 4, 33), 0),
                      ((399, 1, 64), 0), ((400, 5, 64), 64), ((400, 5, 64), 16), ((130, 5, 33), 32),
                      ((399, 1, 64), 7)):
        if cuts == (1, 1, 1) and n_state > 100:
            continue
        slots = [3, 0, 4]
        state[slots] = 0.0
        at = [0] * 3
        rows = [[] for _ in lengths]
        while any(a < n for a, n in zip(at, lengths)):
            live = [i for i in range(3) if at[i] < lengths[i]]
            take = [min(cuts[i], lengths[i] - at[i]) for i in live]
            step = scan_step(take, [slots[i] for i in live])
            cat = lambda j: np.concatenate([seqs[i][j][at[i]:at[i] + t] for i, t in zip(live, take)])
            low = dev(cat(1))
            dt = ops.step_size(low, rank, dev(w_dt, T), dev(b_dt, T))
            close(dt, cat(3), torch.float32, "step sizes")
            if step.is_decode:                      # the kernel makes the step sizes itself
                dt = None
            out = ops.selective_scan(dev(cat(0), T), dt, low, rank + 3, rank + 3 + n_state, n_state,
                                     dev(cat(2)), dev(a_log, T), dev(d_skip, T), state, step,
                                     run=0 if dt is None else run,
                                     dt_weight=dev(w_dt, T), dt_bias=dev(b_dt, T))
            for i, t, lo in zip(live, take, np.cumsum([0] + take)):
                rows[i].append(out[lo:lo + t])
                at[i] += t
        for i in range(3):
            close(torch.cat(rows[i]), seqs[i][4], T, f"cuts {cuts}, runs of {run}, sequence {i}")
    # a step that must leave the state as it was (a layer call that does not own its entry)
    before = state.clone()
    step = scan_step([5], [0])
    low = dev(seqs[1][1])
    ops.selective_scan(dev(seqs[1][0], T), ops.step_size(low, rank, dev(w_dt, T), dev(b_dt, T)),
                       low, rank + 3, rank + 3 + n_state, n_state, dev(seqs[1][2]), dev(a_log, T),
                       dev(d_skip, T), state, step, keep_state=False, run=2)
    assert torch.equal(state, before)


# -- attention without softmax over a fading state ---------------------------------------------------

@pytest.mark.parametrize("heads,dim,vdim,decay", [
    (3, 16, 24, (0.5, 0.9, 0.9995)), (2, 24, 8, (0.97, 0.7)), (5, 12, 20, (1.0, 0.3, 0.8, 0.99, 0.6)),
    (1, 36, 28, (0.9,)), (2, 192, 64, (0.98, 0.999)), (4, 64, 128, (0.9, 0.95, 0.99, 0.999))])
def test_fading_state_over_pieces_with_a_token_far_back(heads, dim, vdim, decay):
    """The slowest head's key at token 1 is far larger than any later one, and the last query
    points at it: what the head gives there is that token's value, faded 398 times."""
    rng = np.random.default_rng(dim + vdim)
    lengths = (400, 3, 70)
    eps, out_scale = 1e-5, 0.7
    qk, vc = heads * dim, heads * vdim
    slow = int(np.argmax(decay))
    w = rounded(1 + 0.2 * rng.standard_normal(vc), torch.bfloat16)
    seqs = []
    for n in lengths:
        proj = rng.standard_normal((n, 7 + 2 * qk + 2 * vc))
        if n > 100:
            proj[1, 7 + qk + slow * dim:7 + qk + (slow + 1) * dim] = 20.0
            proj[-1, 7 + slow * dim:7 + (slow + 1) * dim] = 6.0
        proj = dev(proj).cpu().numpy().astype(np.float64)
        q, k, v = (plain.silu(proj[:, lo:lo + c]).reshape(n, heads, -1)
                   for lo, c in ((7, qk), (7 + qk, qk), (7 + 2 * qk, vc)))
        o = np.empty((n, heads, vdim))
        for h in range(heads):
            S = np.zeros((dim, vdim))
            for i in range(n):
                S = decay[h] * S + np.outer(k[i, h], v[i, h])
                o[i, h] = S.T @ q[i, h]
        if n > 100 and decay[slow] > 0.999:
            far = decay[slow] ** (n - 2) * (k[1, slow] @ q[-1, slow]) * v[1, slow]
            assert np.abs(far).max() > 0.5 * np.abs(o[-1, slow]).max()
        o = o.reshape(n, vc)
        seqs.append((proj, o, plain.rms_norm(o, w, eps) * plain.sigmoid(proj[:, 7 + 2 * qk + vc:])
                     * out_scale))
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
            step = scan_step(take, [slots[i] for i in live])
            proj = dev(np.concatenate([seqs[i][0][at[i]:at[i] + t] for i, t in zip(live, take)]))
            y = ops.decay_attention(proj, 7, 7 + qk, 7 + 2 * qk, heads, dim, vdim, less_one, state,
                                    step, run=run)
            out = ops.norm_gate(y, dev(w, torch.bfloat16), proj[:, 7 + 2 * qk + vc:], eps,
                                out_scale, torch.float32)
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
                        scan_step([3], [4]), keep_state=False, run=2)
    assert torch.equal(state, before)
    plain_out = ops.norm_gate(dev(seqs[1][1]), dev(w, torch.bfloat16), None, eps, 1.0, torch.bfloat16)
    close(plain_out, plain.rms_norm(seqs[1][1], w, eps), torch.bfloat16, "no gate")
