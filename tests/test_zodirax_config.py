"""The Zodirax configuration: what it reads, what it refuses, the parts it builds and what they
ask of the cache, and the plain model's own mechanisms on hand-made inputs. No GPU."""

import copy
import math

import numpy as np
import pytest

import plain_zodirax as plain
from semantic_aware_adaptive_kv_cache_precision_b200.cache import KVNeed, MultiNeed, StateNeed
from semantic_aware_adaptive_kv_cache_precision_b200.config import (BandScaling, ConfigError,
                                                                   RotarySpec, config_from_dict,
                                                                   known_architectures)
from semantic_aware_adaptive_kv_cache_precision_b200.engine.model import DecoderModel
from semantic_aware_adaptive_kv_cache_precision_b200.parts import RotaryHalf
from zodirax_configs import CONFIGS, MIXED, ODD, WIDE


def test_registered_and_round_trips():
    assert "Zodirax" in known_architectures()
    for config, _ in CONFIGS.values():
        typed = config_from_dict(copy.deepcopy(config))
        assert config_from_dict(typed.to_dict()) == typed


def test_layers_run_in_the_listed_order_with_a_cache_entry_each():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    assert [c.block for c in spec.run_order] == [0, 1, 2, 3]
    assert [c.cache for c in spec.run_order] == [0, 1, 2, 3]
    assert [b.mixer.kind for b in spec.blocks] == ["parallel_mixer", "selective_scan",
                                                  "selective_scan", "parallel_mixer"]
    assert [b.ffn is None for b in spec.blocks] == [False, True, False, True]
    assert spec.tie_head and spec.embed_scale == 2.5 and spec.final_norm.offset == 1.0
    other = config_from_dict(copy.deepcopy(ODD)).model_spec()
    assert [b.mixer.kind for b in other.blocks] == ["selective_scan", "parallel_mixer",
                                                   "parallel_mixer", "selective_scan"]


def test_declared_tensors_carry_the_configuration_s_sizes():
    spec = config_from_dict(copy.deepcopy(MIXED)).model_spec()
    shapes = {d.name: tuple(d.shape) for d in DecoderModel.tensor_decls_of(spec)}
    assert shapes["embed"] == (211, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.left.q"] == (4 * 32, 96) and shapes["l0.mix.left.q.b"] == (128,)
    assert shapes["l0.mix.left.k"] == (2 * 32, 96) and shapes["l0.mix.left.v"] == (2 * 24, 96)
    assert shapes["l0.mix.left.q.norm"] == (128,) and shapes["l0.mix.left.k.norm"] == (64,)
    assert shapes["l0.mix.left.sink"] == (4,) and shapes["l0.mix.left.o"] == (96, 4 * 24)
    assert shapes["l0.mix.right.q"] == (48, 96) and shapes["l0.mix.right.v"] == (72, 96)
    assert shapes["l0.mix.right.g"] == (72, 96) and shapes["l0.mix.right.norm"] == (72,)
    assert shapes["l0.mix.right.o"] == (96, 72) and shapes["l0.mlp.down"] == (96, 80)
    assert shapes["l1.mix.in"] == (256, 96) and shapes["l1.mix.conv"] == (128, 4)
    assert shapes["l1.mix.x"] == (6 + 2 * 16, 128) and shapes["l1.mix.dt"] == (128, 6)
    assert shapes["l1.mix.A_log"] == (128, 16) and shapes["l1.mix.D"] == (128,)
    assert "l1.mlp.gate" not in shapes and "l1.norm2" not in shapes        # no feed-forward
    assert shapes["l2.mix.conv"] == (72, 2) and shapes["l2.norm2"] == (96,)


def test_what_the_layers_ask_of_the_cache():
    spec = config_from_dict(copy.deepcopy(ODD)).model_spec()
    needs = DecoderModel(spec, "float32", "cpu").cache_needs()
    assert needs[0] == MultiNeed((StateNeed((2, 50), "float32"), StateNeed((50, 7), "float32")))
    assert needs[1] == MultiNeed((KVNeed(2, 20, 3, value_dim=12, keep_first=1),
                                  StateNeed((5, 20, 12), "float32")))
    assert needs[2].parts[0] == KVNeed(1, 24, 100, value_dim=36, keep_first=70)
    assert needs[3] == MultiNeed((StateNeed((0, 30), "float32"), StateNeed((30, 1), "float32")))


def test_problems_are_listed_together():
    bad = copy.deepcopy(MIXED)
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 7
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    bad["layers"][0]["mixer"]["right"]["decay"] = [0.5]
    bad["layers"][1]["mixer"]["state"] = 0
    bad["layers"][2]["type"] = "convolution"
    bad["layers"][3]["mlp"] = {"kind": "sparse", "ff": 8}
    del bad["width"]
    with pytest.raises(ConfigError) as err:
        config_from_dict(bad)
    text = str(err.value)
    for piece in ("rot.dims", "kv_heads", "decay", "mixer.state", "convolution", "mlp.kind",
                  "width"):
        assert piece in text


def test_band_frequencies_by_hand():
    """All three bands occur: wavelengths below original / high stay, above original / low are
    divided by the factor, and between them the two are blended."""
    rot = {"base": 100.0, "dims": 8,
           "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 60}}
    f = plain.stretched_frequencies(rot)
    raw = [100.0 ** (-2 * i / 8) for i in range(4)]
    lengths = [2 * math.pi / x for x in raw]          # 6.3, 19.9, 62.8, 198.7
    assert lengths[0] < 60 / 4.0 < lengths[1] < 60 / 1.0 < lengths[2]
    s = (60 / lengths[1] - 1.0) / (4.0 - 1.0)
    assert f[0] == raw[0] and f[1] == pytest.approx((1 - s) * raw[1] / 4.0 + s * raw[1])
    assert f[2] == raw[2] / 4.0 and f[3] == raw[3] / 4.0
    assert np.array_equal(plain.stretched_frequencies({"base": 100.0, "dims": 8}), raw)
    # the library's table is the same
    part = RotaryHalf(RotarySpec(16, 8, 100.0, 64, scaling=BandScaling(4.0, 60, 1.0, 4.0)), "",
                      "float32")
    got, magnitude = part.frequencies()
    assert np.allclose(got, f, rtol=1e-15) and magnitude == 1.0


def test_who_sees_whom():
    seen = plain.visible(9, 3, 2)
    assert seen[8].tolist() == [True, True, False, False, False, False, True, True, True]
    assert seen[2].tolist() == [True, True, True] + [False] * 6
    assert seen[4].tolist() == [True, True, True, True, True, False, False, False, False]
    assert not plain.visible(5, 1, 0)[4, :4].any() and plain.visible(5, 1, 0)[4, 4]


def test_the_sink_counts_once_and_has_no_value():
    s = np.array([[0.0, 0.0]])
    w = plain.sink_softmax(s, np.array([[True, True]]), 0.0)
    assert np.allclose(w, [[1 / 3, 1 / 3]])
    w = plain.sink_softmax(s, np.array([[True, False]]), math.log(3.0))
    assert np.allclose(w, [[0.25, 0.0]])
    assert np.allclose(plain.sink_softmax(s, np.array([[True, True]]), -1e9), [[0.5, 0.5]])


def test_the_convolution_s_last_column_is_the_current_token():
    x = np.array([[1.0], [10.0], [100.0], [1000.0]])
    y = plain.causal_conv(x, np.array([[3.0, 2.0, 1.0]]), np.array([0.5]))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 1230.5]


def test_the_scan_and_the_fading_state_by_hand():
    x, dt = np.array([[2.0], [3.0]]), np.array([[0.5], [0.25]])
    A, D = np.array([[-1.0, -2.0]]), np.array([10.0])
    B, C = np.array([[1.0, 1.0], [2.0, 0.0]]), np.array([[1.0, 0.0], [1.0, 1.0]])
    y = plain.selective_scan(x, dt, A, B, C, D)
    s0 = np.array([1.0, 1.0])                               # dt x B at the first token
    s1 = np.exp(0.25 * A[0]) * s0 + 0.75 * B[1]
    assert np.allclose(y[:, 0], [s0[0] + 20.0, s1.sum() + 30.0])
    # one head, dim 1, vdim 1, no projections' mixing: S_t = d S_(t-1) + k_t v_t
    t = {"q": np.eye(1), "k": np.eye(1), "v": np.eye(1), "g": np.zeros((1, 1)),
         "norm": np.ones(1), "o": np.eye(1)}
    h = np.array([[1.0], [2.0], [0.5]])
    m = {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5]}
    a = plain.silu(h[:, 0])
    state = [a[0] * a[0], 0.5 * a[0] * a[0] + a[1] * a[1]]
    state.append(0.5 * state[1] + a[2] * a[2])
    out = plain.decayed_linear_attention(h, t, "", m, 0.0)
    o = np.array(state) * a
    assert np.allclose(out[:, 0], o / np.abs(o) * 0.5)      # unit norm of one number, gate 1/2


def test_sizes_differ_between_the_configurations():
    widths = {c["width"] for c, _ in CONFIGS.values()}
    assert len(widths) == len(CONFIGS) and WIDE["layers"][1]["mixer"]["state"] > 128


def test_what_config_json_does_not_give_is_not_applied():
    bare = copy.deepcopy(MIXED)
    mixer = bare["layers"][0]["mixer"]
    for key in ("left_scale", "right_scale"):
        del mixer[key]
    for key in ("scale", "kv_heads", "vdim"):
        del mixer["left"][key]
    del mixer["left"]["rot"]["scaling"], mixer["left"]["mask"]["keep_first"], bare["embedding"]
    spec = config_from_dict(bare).model_spec()
    left, right = spec.blocks[0].mixer.left, spec.blocks[0].mixer.right
    assert (left.out_scale, right.out_scale, left.scale, spec.embed_scale) == (1.0, 1.0, 1.0, 1.0)
    assert (left.kv_heads, left.value_dim, left.keep_first) == (left.heads, left.head_dim, 0)
    assert left.position.scaling is None
