"""Zodirax configurations drawn at random over what config.json allows (widths, the kinds of
layers in any order, head counts, key and value sizes, rotated sizes with and without
stretched wavelengths, windows and kept first tokens, decays, channels, states, taps, ranks,
layers without a feed-forward), each through the engine against the plain model: whole
prompts, the last tokens one by one, and an unequal batch."""

import numpy as np
import pytest

import plain_zodirax as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from helpers import assert_close_to_plain, assert_same_logits
from zodirax_configs import pair, rot, scan

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = np.random.default_rng(2000 + seed)
    pick = lambda options: options[int(rng.integers(len(options)))]
    width = pick([48, 64, 72, 100, 128, 160, 200, 320])

    def ff():
        return None if rng.random() < 0.25 else pick([16, 50, 64, 130, 256])

    layers = []
    for _ in range(int(rng.integers(1, 6))):
        if rng.random() < 0.5:
            layers.append(scan(pick([24, 50, 64, 96, 160, 256]), pick([1, 3, 8, 16, 24, 32, 64, 140]),
                               pick([1, 2, 5, 8, 16, 24]), pick([1, 2, 3, 4, 5, 8]), ff()))
        else:
            kv_heads = pick([1, 2, 3, 4])
            dim = pick([8, 16, 24, 48, 64, 96])
            dims = pick([d for d in (2, 4, 8, 16, 32, 64, 96) if d <= dim])
            scaling = None if rng.random() < 0.3 else (
                float(rng.uniform(1.5, 16)), float(pick([0.5, 1.0, 2.0])), float(pick([3.0, 4.0, 8.0])),
                int(pick([16, 64, 256, 4096])))
            heads = pick([1, 2, 3, 5, 6])
            left = (kv_heads * pick([1, 2, 3]), kv_heads, dim, pick([8, 12, 32, 80, 96]),
                    float(dim ** -0.5 * rng.uniform(0.5, 2)), pick([1, 2, 7, 31, 64, 65, 96, 130, 500]),
                    pick([0, 0, 1, 4, 9, 64, 66]), rot(float(pick([100, 1e4, 3e4, 5e5])), dims, scaling))
            right = (heads, pick([8, 12, 32, 40, 64]), pick([8, 20, 32, 48]),
                     [float(pick([1.0, 0.999, 0.99, 0.9, 0.6, 0.2])) for _ in range(heads)])
            layers.append(pair(left, right, (float(rng.uniform(0.3, 2)), float(rng.uniform(0.3, 2))),
                               ff()))
    return {"architecture": "Zodirax", "vocab": int(rng.integers(50, 700)), "width": width,
            "norm": {"eps": float(pick([1e-6, 1e-5]))},
            "embedding": {"scale": float(pick([1.0, 2.0, 3.0, 0.5]))}, "initializer_range": 0.1,
            "layers": layers}


@pytest.mark.parametrize("seed", range(20))
def test_a_drawn_configuration_in_32_bits(seed, tmp_path):
    config = draw(seed)
    folder = sakv.write_random_model(tmp_path / "m", config, seed, dtype="float32")
    cfg, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype="float32", max_tokens=1024, poison_freed=True).load_weights()
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, config["vocab"], n).astype(np.int64) for n in (170, 37, 2)]
    whole = [engine.forward(p) for p in prompts]
    for got, p in zip(whole, prompts):
        assert_close_to_plain(got, plain.forward(cfg, tensors, p), "float32", f"seed {seed}")
    # the longest prompt again: most of it in one step, its last 40 tokens one by one
    p = prompts[0]
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [p[:130]], [list(range(130))]).cpu().numpy()]
    for t in range(130, len(p)):
        rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
    engine.close([slot])
    assert_same_logits(np.concatenate(rows), whole[0], "float32", f"seed {seed}: decoded")
    # the three together, then decoded together until each ends
    slots = engine.open(3)
    heads = [len(q) - k for q, k in zip(prompts, (5, 3, 1))]
    out = engine.step(slots, [q[:h] for q, h in zip(prompts, heads)],
                      [list(range(h)) for h in heads]).cpu().numpy()
    got = [[out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
    fed = list(heads)
    live = [0, 1, 2]
    while live:
        out = engine.step([slots[i] for i in live], [prompts[i][fed[i]:fed[i] + 1] for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1].cpu().numpy())
            fed[i] += 1
        done = [i for i in live if fed[i] == len(prompts[i])]
        if done:
            engine.close([slots[i] for i in done])
        live = [i for i in live if fed[i] < len(prompts[i])]
    for i in range(3):
        assert_same_logits(np.concatenate(got[i]), whole[i], "float32",
                           f"seed {seed}: request {i} of the batch")
    engine.cache.check()
    assert engine.graph_failure is None


@pytest.mark.parametrize("seed", range(20))
def test_a_drawn_configuration_in_16_bits(seed, tmp_path):
    """A prompt long enough for the recurrent layers to walk it in runs, then tokens one by
    one; judged by the median row within a tenth of its spread, since a drawn configuration
    may be deep (each layer carries its sublayers' rounding to the stream at full size through
    the norms on their outputs) or badly conditioned."""
    config = draw(seed)
    folder = sakv.write_random_model(tmp_path / "m", config, seed, dtype="bfloat16")
    cfg, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype="bfloat16", max_tokens=1024, poison_freed=True).load_weights()
    p = np.random.default_rng(seed).integers(0, config["vocab"], 330).astype(np.int64)
    want = plain.forward(cfg, tensors, p)
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [p[:290]], [list(range(290))]).cpu().numpy()]
    for t in range(290, len(p)):
        rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
    engine.close([slot])
    got = np.concatenate(rows)
    assert np.isfinite(got).all()
    worst = np.abs(got - want).max(axis=-1) / want.std(axis=-1)
    assert np.median(worst[:290]) <= 0.1, f"seed {seed}: the prompt's median row {np.median(worst[:290]):.3f}"
    assert np.median(worst[290:]) <= 0.1, f"seed {seed}: the decoded median row {np.median(worst[290:]):.3f}"
    assert engine.graph_failure is None
