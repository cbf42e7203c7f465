"""The Gesuvik configuration: what it reads, what it refuses, the parts it builds and what they
ask of the cache, and the plain model's own mechanisms on hand-made inputs. No GPU."""

import copy
import math

import numpy as np
import pytest

import plain_gesuvik as plain
from semantic_aware_adaptive_kv_cache_precision_b200.cache import KVNeed, StateNeed
from semantic_aware_adaptive_kv_cache_precision_b200.config import (ConfigError, RampScaling,
                                                                   RotarySpec, config_from_dict,
                                                                   known_architectures)
from semantic_aware_adaptive_kv_cache_precision_b200.engine.model import DecoderModel
from semantic_aware_adaptive_kv_cache_precision_b200.parts import RotaryHalf
from gesuvik_configs import CONFIGS, MIXED, ODD, WIDE


def test_registered_and_round_trips():
    assert "Gesuvik" in known_architectures()
    for config, _ in CONFIGS.values():
        typed = config_from_dict(copy.deepcopy(config))
        assert config_from_dict(typed.to_dict()) == typed


def test_a_layer_with_another_s_weights_is_one_more_call_of_its_block():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    assert [c.block for c in spec.run_order] == [0, 1, 2, 0, 3]
    assert [c.cache for c in spec.run_order] == [0, 1, 2, 3, 4]
    assert [b.prefix for b in spec.blocks] == ["l0.", "l1.", "l2.", "l4."]
    assert [b.mixer.kind for b in spec.blocks] == ["latent_attention", "decay_attention",
                                                  "window_sink_attention", "decay_attention"]
    assert [b.ffn is None for b in spec.blocks] == [False, True, False, False]
    assert not spec.tie_head and spec.logit_scale == 1.5 and spec.logit_softcap == 20.0
    other = config_from_dict(copy.deepcopy(ODD)).model_spec()
    assert [c.block for c in other.run_order] == [0, 1, 0, 2, 3, 1]
    assert other.logit_scale == 1.0 and other.logit_softcap == 9.0
    assert config_from_dict(copy.deepcopy(WIDE)).model_spec().logit_softcap is None


def test_the_parts_descriptions_carry_the_design_s_constants():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    latent, fading, attention = (spec.blocks[i].mixer for i in (0, 1, 2))
    assert latent.window == 37 and latent.sink and latent.head_gate and latent.q_rank is None
    assert latent.position.kind == "rotary_interleaved" and latent.position.rotary_dim == 8
    assert fading.activation is None and fading.norm == "head" and not fading.norm_weight
    assert fading.gate_kind == "silu" and fading.key_scale == 16 ** -0.5
    assert fading.position.kind == "rotary_half" and fading.position.rotary_dim == 8
    assert attention.qk_norm == "whole" and not attention.bias and attention.keep_first == 0
    assert attention.sink and attention.window == 64
    assert attention.position.scaling == RampScaling(4.0, 64, 8.0, 2.0, 0.1)
    ffn = spec.blocks[0].ffn
    assert (ffn.experts, ffn.identity, ffn.top) == (6, 2, 2) and ffn.score == "softmax"
    assert ffn.correction and not ffn.weight_input and not ffn.shared_gate and not ffn.renormalize
    assert ffn.expert.alpha == 1.702 and ffn.shared.limit == 3.0 and ffn.expert.limit == 1.0
    assert spec.blocks[3].ffn.shared is None


def test_declared_tensors_carry_the_configuration_s_sizes():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    shapes = {d.name: tuple(d.shape) for d in DecoderModel.tensor_decls_of(spec)}
    assert shapes["embed"] == (211, 96) and shapes["head"] == (211, 96)
    assert shapes["final.norm"] == (96,) and shapes["l0.norm1"] == (96,)
    assert shapes["l0.mix.q"] == (4 * 24, 96) and shapes["l0.mix.g"] == (4, 96)
    assert shapes["l0.mix.dkv"] == (48, 96) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (64, 40) and shapes["l0.mix.uv"] == (96, 40)
    assert shapes["l0.mix.sink"] == (4,) and shapes["l0.mix.o"] == (96, 96)
    assert shapes["l0.mlp.router"] == (8, 96) and shapes["l0.mlp.correction"] == (8,)
    assert shapes["l0.mlp.e5.down"] == (96, 48) and "l0.mlp.e6.down" not in shapes
    assert shapes["l0.mlp.shared.gate"] == (32, 96) and "l0.mlp.shared.sg" not in shapes
    assert shapes["l1.mix.q"] == (48, 96) and shapes["l1.mix.v"] == (72, 96)
    assert shapes["l1.mix.g"] == (72, 96) and shapes["l1.mix.o"] == (96, 72)
    assert "l1.mix.norm" not in shapes and "l1.norm2" not in shapes and "l1.mlp.router" not in shapes
    assert shapes["l2.mix.q"] == (128, 96) and shapes["l2.mix.k"] == (64, 96)
    assert shapes["l2.mix.v"] == (48, 96) and shapes["l2.mix.q.norm"] == (128,)
    assert shapes["l2.mix.k.norm"] == (64,) and "l2.mix.q.b" not in shapes
    assert not any(name.startswith("l3.") for name in shapes)         # another layer's weights
    assert shapes["l4.mlp.router"] == (4, 96) and "l4.mlp.shared.gate" not in shapes


def test_what_the_layers_ask_of_the_cache():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    needs = DecoderModel(spec, "float32", "cpu").cache_needs()
    assert needs[0] == KVNeed(1, 48, 37, value_dim=0) and needs[3] == needs[0]
    assert needs[1] == StateNeed((3, 24, 16), "float32")
    assert needs[2] == KVNeed(2, 32, 64, value_dim=24)
    assert needs[4] == StateNeed((2, 8, 24), "float32")
    odd = DecoderModel(config_from_dict(copy.deepcopy(ODD)).model_spec(), "float32", "cpu")
    assert odd.cache_needs()[4] == KVNeed(3, 24, None, value_dim=36)
    assert odd.cache_needs()[5] == odd.cache_needs()[1]


def test_every_problem_is_named_at_once():
    bad = copy.deepcopy(MIXED)
    bad["width"] = 0
    bad["layers"][0]["mixer"]["rot_dim"] = 7
    bad["layers"][1]["mixer"]["decay"] = [0.5]
    bad["layers"][2]["mixer"]["kv_heads"] = 3
    bad["layers"][2]["mlp"]["router"]["top"] = 9
    bad["layers"][3]["weights_of"] = 1
    bad["layers"][4]["type"] = "mamba"
    with pytest.raises(ConfigError) as err:
        config_from_dict(bad)
    text = str(err.value)
    for piece in ("width", "rot_dim", "decay", "kv_heads", "router.top", "weights_of", "'mamba'"):
        assert piece in text, piece
    for source in (3, 5, -1, "0"):        # itself, beyond the list, before it, not a number
        bad = copy.deepcopy(MIXED)
        bad["layers"][3]["weights_of"] = source
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_stretched_frequencies_by_hand_and_in_the_library_s_table():
    turn = {"base": 10000.0, "dims": 16,
            "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    f, size = plain.frequencies(turn)
    # p(t) = 16 ln(64 / (2 pi t)) / (2 ln 10000): p(8) = 0.21, p(2) = 1.41 -> lo 0, hi 2
    plain_f = np.array([10000.0 ** (-2 * i / 16) for i in range(8)])
    ramp = np.clip(np.arange(8) / 2.0, 0, 1)
    assert np.allclose(f, plain_f / 4 * ramp + plain_f * (1 - ramp), rtol=1e-14)
    assert f[0] == 1.0 and math.isclose(f[1], plain_f[1] * (0.5 / 4 + 0.5)) and f[7] == plain_f[7] / 4
    assert math.isclose(size, 0.1 * math.log(4.0) + 1.0)
    part = RotaryHalf(RotarySpec(32, 16, 10000.0, 64, scaling=RampScaling(4.0, 64, 8.0, 2.0)),
                      "", "float32")
    got, magnitude = part.frequencies()
    assert np.allclose(got, f, rtol=1e-14) and math.isclose(magnitude, size)
    plain_turn = {"base": 10000.0, "dims": 16}
    assert plain.frequencies(plain_turn)[1] == 1.0
    assert np.array_equal(plain.frequencies(plain_turn)[0], plain_f)


def test_the_two_pairings_turn_a_pair_by_the_position_s_angle():
    turn = {"base": 100.0, "dims": 4}
    x = np.zeros((1, 1, 6))
    x[0, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    a0, a1 = 7 * 1.0, 7 * 100.0 ** -0.5
    halves = plain.turn_halves(x, [7], turn)[0, 0]
    assert np.allclose(halves, [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1),
                                5.0, 6.0])
    near = plain.turn_neighbours(x, [7], turn)[0, 0]
    assert np.allclose(near, [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
                              3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1),
                              5.0, 6.0])
    assert np.array_equal(plain.turn_halves(x, [0], turn), x)


def test_who_sees_whom_and_the_sink():
    seen = plain.banded(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True]
    assert seen[1].tolist() == [True, True, False, False, False, False]
    assert plain.banded(4, None)[3].all() and not plain.banded(4, 1)[3, 2]
    s = np.array([[0.0, 0.0], [1.0, 2.0]])
    w = plain.sink_softmax(s, plain.banded(2, None), math.log(2.0))
    assert np.allclose(w[0], [1 / 3, 0.0])               # exp(0) / (exp(0) + 2)
    assert np.allclose(w[1], np.exp([1.0, 2.0]) / (math.e + math.e ** 2 + 2.0))
    assert np.allclose(plain.sink_softmax(s, plain.banded(2, None), None)[1].sum(), 1.0)


def test_retention_by_hand():
    """One head, two numbers a key, one a value, no rotation: S after token 1 is decay k0 v0 +
    k1 v1, and the head's output over its root mean square is a sign."""
    t = {"q": np.eye(2), "k": np.eye(2), "v": np.array([[1.0, 1.0]]), "g": np.array([[1.0, 0.0]]),
         "o": np.array([[2.0], [0.0]])}
    m = {"heads": 1, "dim": 2, "vdim": 1, "decay": [0.5]}
    h = np.array([[1.0, 0.0], [0.0, 2.0], [3.0, -5.0]])
    # k = h / sqrt(2), v = h0 + h1: S = [sum decay^(i-j) k_j v_j]; o_i = q_i . S
    k, v = h / math.sqrt(2), h.sum(1)
    S1 = 0.5 * k[0] * v[0] + k[1] * v[1]
    S2 = 0.5 * S1 + k[2] * v[2]
    raw = np.array([k[0] @ h[0] * v[0], S1 @ h[1], S2 @ h[2]])
    want = raw / np.sqrt(raw ** 2 + 1e-6) * plain.silu(h[:, 0])
    got = plain.retention(h, t, "", m, 1e-6)
    assert np.allclose(got[:, 0], 2.0 * want) and np.allclose(got[:, 1], 0.0)


def test_routing_by_hand():
    """Four outputs of which the last is an identity expert; the correction lifts output 1 over
    output 0 for the choice, and the weight stays the softmax's."""
    t = {"router": np.array([[2.0], [1.0], [0.0], [3.0]]), "correction": np.array([0.0, 0.5, 0.0, 0.0])}
    h = np.array([[1.0]])
    chosen, weights = plain.route(h, t, "", 2)
    s = np.exp([2.0, 1.0, 0.0, 3.0]) / np.exp([2.0, 1.0, 0.0, 3.0]).sum()
    assert s[0] > s[1] and s[1] + 0.5 > s[0]
    assert chosen.tolist() == [[3, 1]] and np.allclose(weights, [[s[3], s[1]]])
    for e in range(3):
        t[f"e{e}.gate"], t[f"e{e}.up"] = np.array([[5.0]]), np.array([[-9.0]])
        t[f"e{e}.down"] = np.array([[float(e + 1)]])
    mlp = {"router": {"experts": 3, "identity": 1, "top": 2}, "expert": {"ff": 1, "limit": 2.0}}
    # expert 1: g = min(5, 2) = 2, u = clamp(-9) = -2, y = 2 sigmoid(3.404) (-1), times down = 2
    y = 2.0 * plain.sigmoid(1.702 * 2.0) * (-2.0 + 1.0)
    assert np.allclose(plain.experts(h, t, "", mlp), s[3] * 1.0 + s[1] * 2.0 * y)
