"""Gesuvik: a pre-norm decoder whose layers are listed one by one in config.json; a layer may
run with another layer's weights and a cache of its own.

    {"architecture": "Gesuvik", "vocab": V, "width": W, "norm": {"eps": e},
     "logit_scale": a, "logit_softcap": c,
     "layers": [{"type": "retention",
                 "mixer": {"heads": H, "dim": D, "vdim": Dv, "decay": [...],
                           "rot": {"base": b, "dims": R}},
                 "mlp": {"kind": "moe", "router": {"experts": E, "identity": I, "top": k},
                         "expert": {"ff": F, "limit": l}, "shared": {"ff": Fs, "limit": ls}}},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": C,
                           "scale": s, "mask": {"size": w}, "rot": {"base": b, "dims": R}},
                 "mlp": {...}},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s,
                           "mask": {"size": w},
                           "rot": {"base": b, "dims": R,
                                   "scaling": {"factor": f, "original": n, "fast": x, "slow": y}}},
                 "mlp": null},
                {"type": "latent_attention", "weights_of": 1, "mixer": {...}, "mlp": {...}}]}

A layer is `x += mixer(norm1(x)); x += ffn(norm2(x))` with RMS norms (`BlockSpec`). Its mixer is
retention, a fading state a head with turned queries and keys, a norm a head and a silu gate
(`DecayAttentionSpec`); attention over one cached latent a position with a shared key part
turned in pairs of neighbours, a window, a sink and a gate a head (`LatentAttentionSpec`); or
grouped-query attention with queries and keys normed over their whole projection, a partial
rotation with stretched wavelengths, a window and a sink (`WindowSinkAttentionSpec`). Its
feed-forward is a mixture of clamped gated experts chosen by a softmax router with a
correction for the choice, identity experts and a shared expert (`RoutedExpertsSpec`), or
absent. A layer with `weights_of: j` has no tensors: it is one more call of layer j's block
with a cache entry of its own (`LayerCall`). The logits are multiplied by `logit_scale` and
bent by `logit_softcap`. Tensors: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`,
`l<i>.mlp.*`, `final.norm`, `head`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import (BlockSpec, ClampedExpertSpec, ConfigError, DecayAttentionSpec,
                    LatentAttentionSpec, LayerCall, ModelSpec, NormSpec, RampScaling, RotarySpec,
                    RoutedExpertsSpec, WindowSinkAttentionSpec)

#: positions the rotation's table may be asked for; a sequence is bounded by the cache
MAX_POSITIONS = 1 << 22
#: the activation's constant in an expert: y = g * sigmoid(ALPHA * g) * (u + 1)
EXPERT_ALPHA = 1.702
#: cosines and sines of a stretched rotation are multiplied by SLOPE * ln(factor) + 1
MAGNITUDE_SLOPE = 0.1

KINDS = ("retention", "latent_attention", "attention")


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class GesuvikLayer:
    type: str                       # one of KINDS
    mixer: dict                     # the entry's own keys, checked
    mlp: Optional[dict]             # None: no feed-forward
    weights_of: Optional[int]       # the layer whose tensors this one uses (None: its own)


@dataclass(frozen=True)
class GesuvikConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    initializer_range: float = 0.05

    architecture = "Gesuvik"

    @classmethod
    def from_dict(cls, raw: dict) -> "GesuvikConfig":
        problems = []

        def positive_int(where, holder, key):
            v = holder.get(key) if isinstance(holder, dict) else None
            if not _is_int(v) or v <= 0:
                problems.append(f"{where}{key}: expected a positive integer, config.json has {v!r}")
                return 1
            return v

        def number(where, holder, key, low=None):
            v = holder.get(key) if isinstance(holder, dict) else None
            if not _is_number(v) or (low is not None and v <= low):
                problems.append(f"{where}{key}: expected a number"
                                + (f" above {low}" if low is not None else "")
                                + f", config.json has {v!r}")
                return 1.0
            return float(v)

        def rotation(where, m, most, scaling_allowed):
            rot = m.get("rot")
            if rot is None:
                return None
            dims = positive_int(where + "rot.", rot, "dims")
            if dims % 2 or dims > most:
                problems.append(f"{where}rot.dims: {dims} must be even and at most {most}")
            out = {"base": number(where + "rot.", rot, "base", 0.0), "dims": dims}
            sc = rot.get("scaling") if isinstance(rot, dict) else None
            if sc is not None:
                if not scaling_allowed:
                    problems.append(f"{where}rot.scaling: not built for this mixer")
                sw = where + "rot.scaling."
                out["scaling"] = {k: number(sw, sc, k, 0.0)
                                  for k in ("factor", "original", "fast", "slow")}
            return out

        def window(where, m):
            mask = m.get("mask")
            return None if mask is None else {"size": positive_int(where + "mask.", mask, "size")}

        vocab = positive_int("", raw, "vocab")
        width = positive_int("", raw, "width")
        eps = (raw.get("norm") or {}).get("eps")
        if not _is_number(eps) or eps < 0:
            problems.append(f"norm.eps: expected a number >= 0, config.json has {eps!r}")
            eps = 0.0
        logit_scale = 1.0 if raw.get("logit_scale") is None else number("", raw, "logit_scale")
        softcap = None if raw.get("logit_softcap") is None \
            else number("", raw, "logit_softcap", 0.0)
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            problems.append("layers: expected a list of layers")
            listed = []
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                problems.append(f"{where}mixer: expected an object with the mixer's sizes")
                continue
            kind, m, mw = entry.get("type"), entry["mixer"], where + "mixer."
            if kind not in KINDS:
                problems.append(f"{where}type: {kind!r} is none of {', '.join(KINDS)}")
                continue
            mixer = {k: positive_int(mw, m, k) for k in ("heads", "dim")}
            mixer["vdim"] = mixer["dim"] if m.get("vdim") is None else positive_int(mw, m, "vdim")
            if kind == "retention":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != mixer["heads"] \
                        or not all(_is_number(d) for d in decay):
                    problems.append(f"{mw}decay: expected one number for each of the "
                                    f"{mixer['heads']} heads, config.json has {decay!r}")
                    decay = [1.0] * mixer["heads"]
                mixer["decay"] = [float(d) for d in decay]
                mixer["rot"] = rotation(mw, m, mixer["dim"], False)
                if mixer["dim"] > 256:
                    problems.append(f"{mw}dim up to 256 is what the recurrence kernel takes")
            elif kind == "latent_attention":
                mixer["rot_dim"] = positive_int(mw, m, "rot_dim")
                mixer["kv_rank"] = positive_int(mw, m, "kv_rank")
                if mixer["rot_dim"] % 2:
                    problems.append(f"{mw}rot_dim: {mixer['rot_dim']} must be even")
                if mixer["kv_rank"] > 512 or mixer["kv_rank"] + mixer["rot_dim"] > 640:
                    problems.append(f"{mw}kv_rank up to 512 and kv_rank + rot_dim up to 640 are "
                                    "what the attention kernel takes")
                mixer["scale"] = (mixer["dim"] + mixer["rot_dim"]) ** -0.5 \
                    if m.get("scale") is None else number(mw, m, "scale")
                mixer["mask"] = window(mw, m)
                rot = rotation(mw, m, 1 << 30, False)
                if rot is None:
                    problems.append(f"{mw}rot: the shared key part needs a rotation's base")
                    rot = {"base": 10000.0}
                # (the rotated vector is the rot_dim part, whatever rot.dims says)
                mixer["rot"] = {"base": rot["base"], "dims": mixer["rot_dim"]}
            else:
                mixer["kv_heads"] = mixer["heads"] if m.get("kv_heads") is None \
                    else positive_int(mw, m, "kv_heads")
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{mw}{mixer['heads']} heads are not a multiple of "
                                    f"{mixer['kv_heads']} kv_heads")
                if mixer["dim"] > 640 or mixer["vdim"] > 512:
                    problems.append(f"{mw}dim up to 640 and vdim up to 512 are what the attention "
                                    "kernel takes")
                mixer["scale"] = mixer["dim"] ** -0.5 if m.get("scale") is None \
                    else number(mw, m, "scale")
                mixer["mask"] = window(mw, m)
                mixer["rot"] = rotation(mw, m, mixer["dim"], True)
            mlp = entry.get("mlp")
            if mlp is not None:
                lw = where + "mlp."
                if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
                    problems.append(f"{lw}kind: only 'moe' is built, config.json has {mlp!r}")
                    mlp = None
                else:
                    r = mlp.get("router")
                    router = {"experts": positive_int(lw + "router.", r, "experts"),
                              "top": positive_int(lw + "router.", r, "top")}
                    identity = r.get("identity", 0) if isinstance(r, dict) else 0
                    if not _is_int(identity) or identity < 0:
                        problems.append(f"{lw}router.identity: expected an integer >= 0, "
                                        f"config.json has {identity!r}")
                        identity = 0
                    router["identity"] = identity
                    if router["top"] > router["experts"] + identity:
                        problems.append(f"{lw}router.top: more than the router's outputs")
                    e = mlp.get("expert")
                    out = {"kind": "moe", "router": router,
                           "expert": {"ff": positive_int(lw + "expert.", e, "ff"),
                                      "limit": number(lw + "expert.", e, "limit", 0.0)}}
                    sh = mlp.get("shared")
                    out["shared"] = None if sh is None else {
                        "ff": positive_int(lw + "shared.", sh, "ff"),
                        "limit": number(lw + "shared.", sh, "limit", 0.0)}
                    mlp = out
            source = entry.get("weights_of")
            if source is not None:
                if not _is_int(source) or not 0 <= source < len(listed) or source == i \
                        or not isinstance(listed[source], dict) \
                        or listed[source].get("weights_of") is not None \
                        or listed[source].get("type") != kind:
                    problems.append(f"{where}weights_of: expected the index of another layer "
                                    f"of type {kind!r} with tensors of its own, config.json has "
                                    f"{source!r}")
                    source = None
            layers.append(GesuvikLayer(kind, mixer, mlp, source))
        if problems:
            raise ConfigError("config.json cannot describe a Gesuvik model:\n    "
                              + "\n    ".join(problems))
        return cls(vocab=vocab, width=width, eps=float(eps), layers=tuple(layers),
                   logit_scale=logit_scale, logit_softcap=softcap,
                   initializer_range=float(raw.get("initializer_range", 0.05)))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""

        def pruned(v):
            if isinstance(v, dict):
                return {k: pruned(x) for k, x in v.items() if x is not None}
            return v

        layers = []
        for layer in self.layers:
            entry = {"type": layer.type, "mixer": pruned(layer.mixer),
                     "mlp": None if layer.mlp is None else pruned(layer.mlp)}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.eps}, "logit_scale": self.logit_scale, "layers": layers,
               "initializer_range": self.initializer_range}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out

    # -- the parts' descriptions -----------------------------------------------------------

    def _rotary(self, m, head_dim, kind="rotary_half"):
        rot = m.get("rot")
        if rot is None:
            return None
        sc = rot.get("scaling")
        return RotarySpec(
            head_dim=head_dim, rotary_dim=rot["dims"], theta=rot["base"],
            max_positions=MAX_POSITIONS, kind=kind,
            scaling=None if sc is None else RampScaling(
                factor=sc["factor"], original=sc["original"], fast=sc["fast"], slow=sc["slow"],
                magnitude_slope=MAGNITUDE_SLOPE))

    def _mixer(self, layer):
        m, kind = layer.mixer, layer.type
        window = None if m.get("mask") is None else m["mask"]["size"]
        if kind == "retention":
            return DecayAttentionSpec(
                hidden=self.width, heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"],
                decay=tuple(m["decay"]), eps=self.eps, activation=None,
                position=self._rotary(m, m["dim"]), key_scale=m["dim"] ** -0.5, norm="head",
                norm_weight=False, gate_kind="silu")
        if kind == "latent_attention":
            return LatentAttentionSpec(
                hidden=self.width, heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                value_dim=m["vdim"], kv_rank=m["kv_rank"], q_rank=None, scale=m["scale"],
                eps=self.eps, position=self._rotary(m, m["rot_dim"], "rotary_interleaved"),
                window=window, sink=True, head_gate=True)
        return WindowSinkAttentionSpec(
            hidden=self.width, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"],
            value_dim=m["vdim"], scale=m["scale"], window=window, keep_first=0, eps=self.eps,
            position=self._rotary(m, m["dim"]), sink=True, qk_norm="whole", bias=False)

    def _ffn(self, layer):
        mlp = layer.mlp
        if mlp is None:
            return None
        shared = mlp.get("shared")
        return RoutedExpertsSpec(
            hidden=self.width, experts=mlp["router"]["experts"], top=mlp["router"]["top"],
            expert=ClampedExpertSpec(mlp["expert"]["ff"], mlp["expert"]["limit"], EXPERT_ALPHA),
            shared=None if shared is None else ClampedExpertSpec(shared["ff"], shared["limit"],
                                                                EXPERT_ALPHA),
            shared_gate=False, score="softmax", renormalize=False, weight_input=False,
            correction=True, identity=mlp["router"]["identity"])

    def run_order(self) -> tuple:
        """One call a layer, each with a cache entry of its own; a layer that uses another's
        weights calls that layer's block."""
        block_of, order = {}, []
        for i, layer in enumerate(self.layers):
            if layer.weights_of is None:
                block_of[i] = len(block_of)
        for i, layer in enumerate(self.layers):
            owner = i if layer.weights_of is None else layer.weights_of
            order.append(LayerCall(block=block_of[owner], cache=i))
        return tuple(order)

    def model_spec(self) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.eps, suffix="")
        blocks, ignore = [], []
        for i, layer in enumerate(self.layers):
            if layer.weights_of is not None:
                continue
            ffn = self._ffn(layer)
            if ffn is None:        # a checkpoint may still carry the absent sublayer's norm
                ignore.append(f"l{i}.norm2")
            blocks.append(BlockSpec(
                prefix=f"l{i}.", mixer=self._mixer(layer), mixer_norm=norm, ffn=ffn,
                ffn_norm=None if ffn is None else norm, mixer_name="mix", ffn_name="mlp",
                mixer_norm_name="norm1", ffn_norm_name="norm2"))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width,
            blocks=tuple(blocks), run_order=self.run_order(), final_norm=norm, tie_head=False,
            max_positions=MAX_POSITIONS, embed_name="embed", final_norm_name="final.norm",
            head_name="head", stored_dtype="bfloat16", init_std=self.initializer_range,
            logit_scale=self.logit_scale, logit_softcap=self.logit_softcap,
            ignore_tensors=tuple(ignore))


register_architecture(GesuvikConfig.architecture, GesuvikConfig)
