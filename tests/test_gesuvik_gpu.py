"""Gesuvik models with random weights through the engine, against the plain model: whole
prompts and the stream after every layer, pieces of prompts down to two tokens, the last
tokens one by one, unequal batches whose slots, cache blocks and states are used again, long
decoding past every window's edge and past block borders, greedy generation through
`Engine.generate`, the trace-replay program and the command line."""

import copy

import numpy as np
import pytest

import plain_gesuvik as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from helpers import assert_same_logits
from gesuvik_configs import CONFIGS, rows_agree

pytestmark = pytest.mark.gpu

def config_for(name, dtype):
    """The configuration as it is for float32. In bfloat16 a token's router scores are off by
    rounding, which now and then turns a choice between two experts of nearly equal score; such
    a row then differs by much, and no margin taken from the exact model says which rows those
    are. So the bfloat16 runs choose every output of the router for every token (the weights
    still are the softmax's); choosing is tested in float32 here and in both types at the
    kernels."""
    config = copy.deepcopy(CONFIGS[name][0])
    if dtype == "bfloat16":
        for layer in config["layers"]:
            if layer["mlp"] is not None:
                r = layer["mlp"]["router"]
                r["top"] = r["experts"] + r["identity"]
    return config


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gesuvik")
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[name, dtype] = sakv.write_random_model(
                root / f"{name}_{dtype}", config_for(name, dtype), CONFIGS[name][1], dtype=dtype)
        return made[name, dtype]

    return get


def prompts_of(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[name][0]["vocab"], n).astype(np.int64) for n in lengths]


def compare(got, want, dtype, what, same=False):
    """`got` against `want`: the plain model's logits, or with `same` another run of the
    engine, which in float32 is equal to the bit."""
    if dtype == "float32" and same:
        assert_same_logits(np.asarray(got), np.asarray(want), dtype, what)
    else:
        rows_agree(got, want, dtype, what)


def setup(folders, name, dtype, max_tokens=1024):
    folder = folders(name, dtype)
    config, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype=dtype, max_tokens=max_tokens, poison_freed=True)
    return engine.load_weights(), config, tensors


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_every_layer(name, dtype, folders):
    engine, config, tensors = setup(folders, name, dtype)
    for p in prompts_of(name, (1, 2, 63, 201)):
        layers = []
        want = plain.forward(config, tensors, p, layers)
        got, states = engine.forward(p, capture_hidden_states=True)
        compare(got, want, dtype, f"{name}: a prompt of {len(p)}")
        assert states.shape[0] == len(config["layers"]) + 1
        for i, s in enumerate(layers[:-1]):      # the stream after each layer but the last
            rows_agree(states[i + 1], s, dtype, f"{name}: after layer {i}")
    assert engine.graph_failure is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_pieces_of_a_prompt_and_tokens_one_by_one(name, dtype, folders):
    engine, config, tensors = setup(folders, name, dtype)
    (p,) = prompts_of(name, (230,), seed=1)
    whole = engine.forward(p)
    compare(whole, plain.forward(config, tensors, p), dtype, name)
    for pieces in ([2, 3, 59, 1, 64, 65, 7, 29], [128, 2, 100], [1] * 3 + [190] + [1] * 37):
        (slot,) = engine.open(1)
        rows, at = [], 0
        for n in pieces:
            rows.append(engine.step([slot], [p[at:at + n]], [list(range(n))]).cpu().numpy())
            at += n
        engine.close([slot])
        assert at == len(p)
        compare(np.concatenate(rows), whole, dtype, f"{name}: pieces {pieces[:4]}...", same=True)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_a_long_prompt_whole_in_halves_and_beside_a_short_one(name, dtype, folders):
    """Long enough that the retention layers walk it in runs side by side (in bfloat16), and
    that the slowest head still holds the first tokens at the end."""
    engine, config, tensors = setup(folders, name, dtype, max_tokens=2048)
    p, short = prompts_of(name, (610, 30), seed=8)
    want = plain.forward(config, tensors, p)
    whole = engine.forward(p)
    compare(whole, want, dtype, f"{name}: 610 tokens")
    slots = engine.open(2)
    first = engine.step(slots, [p[:321], short], [list(range(321)), list(range(30))]).cpu().numpy()
    rest = engine.step(slots[:1], [p[321:]], [list(range(289))]).cpu().numpy()
    engine.close(slots)
    compare(np.concatenate([first[:321], rest]), whole, dtype, f"{name}: in two steps", same=True)
    compare(first[321:], plain.forward(config, tensors, short), dtype, f"{name}: the short one")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_with_slots_blocks_and_states_used_again(name, dtype, folders):
    """The cache holds exactly one batch, so every batch gets blocks and slots that the batch
    before gave back (blocks filled with NaN when they were freed, states left as they were:
    a slot's state must be zeroed when the slot is taken)."""
    lengths = (150, 9, 77, 1)
    engine, config, tensors = setup(folders, name, dtype, max_tokens=7 * 64)
    prompts = prompts_of(name, lengths, seed=2)
    alone = [engine.forward(p) for p in prompts]
    for g, w in zip(alone, prompts):
        compare(g, plain.forward(config, tensors, w), dtype, name)
    tails = (6, 3, 9, 0)
    for turn in range(3):
        order = [(i + turn) % 4 for i in range(4)]
        if turn == 1:
            spare, *slots = engine.open(5)
            engine.close([spare])
        else:
            slots = engine.open(4)
        heads = [lengths[i] - tails[i] for i in order]
        out = engine.step(slots, [prompts[i][:h] for i, h in zip(order, heads)],
                          [list(range(h)) for h in heads]).cpu().numpy()
        rows = {i: [out[sum(heads[:k]):sum(heads[:k + 1])]] for k, i in enumerate(order)}
        fed = dict(zip(order, heads))
        live = [(i, s) for i, s in zip(order, slots)]
        while True:
            done = [(i, s) for i, s in live if fed[i] == lengths[i]]
            if done:
                engine.close([s for _, s in done])
            live = [(i, s) for i, s in live if fed[i] < lengths[i]]
            if not live:
                break
            out = engine.step([s for _, s in live], [prompts[i][fed[i]:fed[i] + 1] for i, _ in live])
            for k, (i, _) in enumerate(live):
                rows[i].append(out[k:k + 1].cpu().numpy())
                fed[i] += 1
        for i in range(4):
            compare(np.concatenate(rows[i]), alone[i], dtype, f"{name}: turn {turn}, request {i}",
                    same=True)
        engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_long_decoding_past_window_edges_and_block_borders(name, dtype, folders):
    """Windows of 3, 37, 64 and 100 positions pass over decoded tokens; the blocks behind them
    go back to the pool."""
    engine, config, tensors = setup(folders, name, dtype, max_tokens=512)
    (p,) = prompts_of(name, (300,), seed=3)
    want = plain.forward(config, tensors, p)
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [p[:5]], [list(range(5))]).cpu().numpy()]
    for t in range(5, len(p)):
        rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
    group = engine.cache.groups[0]
    held = int((group.tables[slot] >= 0).sum())
    assert held < -(-len(p) // 64), "no block behind the window was given back"
    engine.close([slot])
    compare(np.concatenate(rows), want, dtype, f"{name}: 295 tokens one by one")
    assert engine.graph_failure is None


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_engine(name, folders):
    engine, config, tensors = setup(folders, name, "float32")
    prompts = [p.tolist() for p in prompts_of(name, (7, 40, 1), seed=4)]
    got = engine.generate(prompts, 12, stop_at_eos=False)
    for p, g in zip(prompts, got):
        assert g.tolist() == plain.generate(config, tensors, p, 12)
    assert all(e.state == sakv.COMPLETE for e in engine.endings)
    engine.cache.check()
    assert engine.cache.slots.held == 0


def test_generation_in_bfloat16_follows_the_plain_model(folders):
    engine, config, tensors = setup(folders, "mixed", "bfloat16")
    prompts = [p.tolist() for p in prompts_of("mixed", (33, 5), seed=5)]
    got = engine.generate(prompts, 10, stop_at_eos=False)
    for p, g in zip(prompts, got):         # each token is the plain model's choice or a near tie
        ref = plain.forward(config, tensors, p + g.tolist()[:-1])[len(p) - 1:]
        for k, token in enumerate(g.tolist()):
            assert ref[k].max() - ref[k, token] <= 0.2 * ref[k].std()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_runs_a_gesuvik_folder(dtype, folders, tmp_path):
    from test_trace_run_gpu import Trace, entry
    folder = folders("mixed", dtype)
    config, tensors = plain.read_model_folder(folder)
    a, b, c = prompts_of("mixed", (90, 41, 3), seed=6)
    want = {k: plain.forward(config, tensors, p) for k, p in (("a", a), ("b", b), ("c", c))}

    def check(got, request, rows, what):
        compare(got, want[request][np.asarray(rows)], dtype, what)

    trace = Trace(folder, dtype, tmp_path / "out", 512)
    got = trace.send([entry("a", a[:80], range(80)), entry("b", b[:40], [0, 39]),
                      entry("c", c, [2])], end=["c"])
    check(got[:80], "a", range(80), "a's prompt")
    check(got[80:82], "b", [0, 39], "b's prompt")
    check(got[82:], "c", [2], "c")
    got = trace.send([entry("a", a[80:81], [0]), entry("b", b[40:], [0])], end=["b"])
    check(got[:1], "a", [80], "a, one token")
    check(got[1:], "b", [40], "b, one token")
    for t in range(81, 90):
        got = trace.send([entry("a", a[t:t + 1], [0])], end=["a"] if t == 89 else [])
        check(got, "a", [t], f"a alone at {t}")
    trace.finish()


def test_the_command_line_writes_and_runs_a_gesuvik_folder(tmp_path):
    """`random-model` from a config.json, then `generate` and `throughput` on the folder."""
    import json
    from test_cli import run
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["odd"][0]))
    run("random-model", "--config", str(config), "--seed", "3", "--out", str(tmp_path / "m"),
        "--stored-dtype", "float32")
    cfg, tensors = plain.read_model_folder(tmp_path / "m")
    assert cfg["architecture"] == "Gesuvik" and tensors["l0.mlp.router"].shape == (10, 100)
    assert "l2.mix.q" not in tensors and "l5.norm1" not in tensors
    (p,) = prompts_of("odd", (11,), seed=7)
    records, _ = run("generate", "--model", str(tmp_path / "m"), "--dtype", "float32",
                     "--ignore-eos", "--prompt-ids", ",".join(map(str, p)), "--new-tokens", "6")
    assert records[0]["tokens"] == plain.generate(cfg, tensors, p.tolist(), 6)
    records, _ = run("throughput", "--model", str(tmp_path / "m"), "--lengths", "70",
                     "--repeat", "1", "--warmup", "1", "--batch", "2")
    assert records[0]["decode_tokens_per_second"] > 0
