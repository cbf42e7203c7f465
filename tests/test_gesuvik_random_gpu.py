"""Gesuvik configurations drawn at random over what config.json allows (widths, the kinds of
layers in any order, layers that run with an earlier layer's weights, head counts, key, value,
latent and rotated sizes, rotations of a part, of the whole and none, stretched wavelengths,
windows, decays, experts, identity experts, choices, shared experts, layers without a
feed-forward, logit scale and cap), each through the engine against the plain model: whole
prompts, the last tokens one by one, and an unequal batch."""

import copy

import numpy as np
import pytest

import plain_gesuvik as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from helpers import assert_same_logits
from gesuvik_configs import again, attention, latent, moe, retention, rot, rows_agree

pytestmark = pytest.mark.gpu


def draw(seed, all_chosen=False):
    rng = np.random.default_rng(3000 + seed)
    pick = lambda options: options[int(rng.integers(len(options)))]
    width = pick([48, 64, 72, 100, 128, 160, 200, 320])

    def mlp():
        if rng.random() < 0.25:
            return None
        experts, identity = pick([1, 2, 3, 5, 8, 12]), pick([0, 0, 1, 2, 4])
        top = experts + identity if all_chosen else int(rng.integers(1, min(experts + identity, 4) + 1))
        shared = None if rng.random() < 0.4 else (pick([16, 40, 64]), float(pick([0.8, 1.5, 7.0])))
        return moe(experts, identity, top, pick([16, 22, 50, 64, 130]), float(pick([0.7, 1.0, 2.0, 7.0])),
                   shared)

    def window():
        return pick([None, 1, 2, 7, 31, 64, 65, 70, 96, 130, 500])

    layers = []
    for _ in range(int(rng.integers(1, 7))):
        kind = pick(["retention", "latent_attention", "attention", "again"])
        if kind == "again" and layers:
            source = int(rng.integers(len(layers)))
            if "weights_of" not in layers[source]:
                layers.append(again(layers[source], source))
                continue
            kind = "retention"
        if kind in ("retention", "again"):
            heads, dim = pick([1, 2, 3, 5]), pick([8, 12, 32, 40, 64, 96])
            dims = pick([None] + [d for d in (2, 4, 8, 12, 32, 64) if d <= dim])
            layers.append(retention(
                heads, dim, pick([8, 20, 32, 48, 64]),
                [float(pick([1.0, 0.9995, 0.99, 0.9, 0.6, 0.2])) for _ in range(heads)],
                None if dims is None else rot(float(pick([100, 1e4, 1e6])), dims), mlp()))
        elif kind == "latent_attention":
            dim, rot_dim = pick([8, 12, 16, 32, 48]), pick([2, 6, 8, 16, 32])
            layers.append(latent(pick([1, 2, 3, 4, 8, 12]), dim, rot_dim, pick([8, 20, 24, 80]),
                                 pick([8, 24, 36, 96, 128]),
                                 float((dim + rot_dim) ** -0.5 * rng.uniform(0.5, 2)), window(),
                                 float(pick([100, 1e4, 5e5])), mlp()))
        else:
            kv_heads, dim = pick([1, 2, 3, 4]), pick([8, 16, 24, 48, 64, 96])
            dims = pick([None] + [d for d in (2, 4, 8, 16, 24, 32, 64, 96) if d <= dim])
            scaling = None if rng.random() < 0.4 else (
                float(rng.uniform(1.5, 16)), int(pick([16, 64, 256, 2048])), float(pick([8.0, 32.0])),
                float(pick([0.5, 1.0, 2.0])))
            layers.append(attention(kv_heads * pick([1, 2, 3, 4]), kv_heads, dim,
                                    pick([8, 12, 32, 80, 96]),
                                    float(dim ** -0.5 * rng.uniform(0.5, 2)), window(),
                                    None if dims is None else rot(float(pick([100, 1e4, 1e6])), dims,
                                                                  scaling), mlp()))
    config = {"architecture": "Gesuvik", "vocab": int(rng.integers(50, 700)), "width": width,
              "norm": {"eps": float(pick([1e-6, 1e-5]))}, "initializer_range": 0.1,
              "layers": layers}
    if rng.random() < 0.7:
        config["logit_scale"] = float(pick([0.5, 2.0, 3.0]))
    if rng.random() < 0.7:
        config["logit_softcap"] = float(pick([5.0, 15.0, 30.0]))
    return config


@pytest.mark.parametrize("seed", range(24))
def test_a_drawn_configuration_in_32_bits(seed, tmp_path):
    config = draw(seed)
    folder = sakv.write_random_model(tmp_path / "m", copy.deepcopy(config), seed, dtype="float32")
    cfg, tensors = plain.read_model_folder(folder)
    engine = sakv.Engine(folder, dtype="float32", max_tokens=1024, poison_freed=True).load_weights()
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, config["vocab"], n).astype(np.int64) for n in (170, 37, 2)]
    whole = [engine.forward(p) for p in prompts]
    for got, p in zip(whole, prompts):
        rows_agree(got, plain.forward(cfg, tensors, p), "float32", f"seed {seed}")
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


@pytest.mark.parametrize("seed", range(24))
def test_a_drawn_configuration_in_16_bits(seed, tmp_path):
    """A prompt long enough for the retention layers to walk it in runs, then tokens one by
    one; every output of a router chosen for every token (a choice that rounding turns is no
    fault); judged by the median row within a tenth of its spread, since a drawn configuration
    may be deep or badly conditioned."""
    config = draw(seed, all_chosen=True)
    folder = sakv.write_random_model(tmp_path / "m", copy.deepcopy(config), seed, dtype="bfloat16")
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
