"""Zodirax: a decoder whose layers are listed one by one in config.json; every layer's norms
sit on its sublayers' outputs only, and the sublayers read the residual stream itself.

    {"architecture": "Zodirax", "vocab": V, "width": W, "norm": {"eps": e},
     "embedding": {"scale": c},
     "layers": [{"type": "mamba1",
                 "mixer": {"inner": E, "state": N, "dt_rank": R, "conv": taps},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s,
                                    "mask": {"size": w, "keep_first": k},
                                    "rot": {"base": b, "dims": R,
                                            "scaling": {"factor": f, "low": l, "high": h,
                                                        "original": n}}},
                           "right": {"heads": H2, "dim": D2, "vdim": Dv2, "decay": [...]},
                           "left_scale": a, "right_scale": b},
                 "mlp": null}, ...]}

A layer is `x += norm1(mixer(x)); x += norm2(ffn(x))` (`OutputNormBlockSpec`) with RMS norms
whose weights are stored around zero (`NormSpec.offset` 1). Its mixer is the selective scan
(`SelectiveScanSpec`) or two mixers side by side (`ParallelMixerSpec`): attention over a window
that keeps the first tokens, with normed and partly rotated queries and keys and a learned logit
in the softmax's denominator (`WindowSinkAttentionSpec`), beside attention without softmax over
a fading state (`DecayAttentionSpec`). The feed-forward is dense and gated with silu, or
absent. The embedding's rows are multiplied by `embedding.scale`; the output head is the
embedding table without that scale. Tensors: `embed`, `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`, `final.norm`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import (BandScaling, ConfigError, DecayAttentionSpec, GatedMLPSpec, LayerCall,
                    ModelSpec, NormSpec, OutputNormBlockSpec, ParallelMixerSpec, RotarySpec,
                    SelectiveScanSpec, WindowSinkAttentionSpec)

#: positions the rotation's table may be asked for; a sequence is bounded by the cache
MAX_POSITIONS = 1 << 22
#: the norms' weights are stored around zero and used as 1 + w
NORM_OFFSET = 1.0


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class ZodiraxLayer:
    type: str                       # "mamba1" | "parallel"
    mixer: dict                     # the entry's own keys, checked
    mlp: Optional[dict]             # None: no feed-forward


@dataclass(frozen=True)
class ZodiraxConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: tuple
    initializer_range: float = 0.05

    architecture = "Zodirax"

    @classmethod
    def from_dict(cls, raw: dict) -> "ZodiraxConfig":
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

        vocab = positive_int("", raw, "vocab")
        width = positive_int("", raw, "width")
        eps = (raw.get("norm") or {}).get("eps")
        if not _is_number(eps) or eps < 0:
            problems.append(f"norm.eps: expected a number >= 0, config.json has {eps!r}")
            eps = 0.0
        embedding = raw.get("embedding")
        embed_scale = 1.0 if embedding is None else number("embedding.", embedding, "scale")
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
            kind, m = entry.get("type"), entry["mixer"]
            mw = where + "mixer."
            if kind == "mamba1":
                mixer = {k: positive_int(mw, m, k) for k in ("inner", "state", "dt_rank", "conv")}
                if mixer["state"] > 512 or mixer["conv"] > 64:
                    problems.append(f"{mw}state up to 512 and conv up to 64 are what the scan "
                                    "kernels take")
            elif kind == "parallel":
                # (a scale that config.json does not give is not applied)
                mixer = {k: 1.0 if m.get(k) is None else number(mw, m, k)
                         for k in ("left_scale", "right_scale")}
                left, lw = m.get("left"), mw + "left."
                if not isinstance(left, dict):
                    problems.append(f"{lw[:-1]}: expected an object with the attention's sizes")
                    left = {}
                a = {k: positive_int(lw, left, k) for k in ("heads", "dim")}
                a["kv_heads"] = a["heads"] if left.get("kv_heads") is None \
                    else positive_int(lw, left, "kv_heads")
                a["vdim"] = a["dim"] if left.get("vdim") is None else positive_int(lw, left, "vdim")
                if a["heads"] % a["kv_heads"]:
                    problems.append(f"{lw}{a['heads']} heads are not a multiple of "
                                    f"{a['kv_heads']} kv_heads")
                if a["dim"] > 640 or a["vdim"] > 512:
                    problems.append(f"{lw}dim up to 640 and vdim up to 512 are what the attention "
                                    "kernel takes")
                a["scale"] = 1.0 if left.get("scale") is None else number(lw, left, "scale")
                mask = left.get("mask")
                if mask is None:
                    a["mask"] = None
                else:
                    keep = mask.get("keep_first", 0) if isinstance(mask, dict) else None
                    if not _is_int(keep) or keep < 0:
                        problems.append(f"{lw}mask.keep_first: expected an integer >= 0, "
                                        f"config.json has {keep!r}")
                        keep = 0
                    a["mask"] = {"size": positive_int(lw + "mask.", mask, "size"),
                                 "keep_first": keep}
                rot = left.get("rot")
                if rot is None:
                    a["rot"] = None
                else:
                    dims = positive_int(lw + "rot.", rot, "dims")
                    if dims % 2 or dims > a["dim"]:
                        problems.append(f"{lw}rot.dims: {dims} must be even and at most dim "
                                        f"{a['dim']}")
                    turned = {"base": number(lw + "rot.", rot, "base", 0.0), "dims": dims}
                    sc = rot.get("scaling") if isinstance(rot, dict) else None
                    if sc is not None:
                        sw = lw + "rot.scaling."
                        turned["scaling"] = {k: number(sw, sc, k, 0.0)
                                             for k in ("factor", "low", "high", "original")}
                        if turned["scaling"]["low"] == turned["scaling"]["high"]:
                            problems.append(f"{sw}low and high must differ")
                    a["rot"] = turned
                mixer["left"] = a
                right, rw = m.get("right"), mw + "right."
                if not isinstance(right, dict):
                    problems.append(f"{rw[:-1]}: expected an object with the sizes of the "
                                    "attention without softmax")
                    right = {}
                b = {k: positive_int(rw, right, k) for k in ("heads", "dim")}
                b["vdim"] = b["dim"] if right.get("vdim") is None else positive_int(rw, right, "vdim")
                decay = right.get("decay")
                if not isinstance(decay, list) or len(decay) != b["heads"] \
                        or not all(_is_number(d) for d in decay):
                    problems.append(f"{rw}decay: expected one number for each of the "
                                    f"{b['heads']} heads, config.json has {decay!r}")
                    decay = [1.0] * b["heads"]
                b["decay"] = [float(d) for d in decay]
                if b["dim"] > 256:
                    problems.append(f"{rw}dim up to 256 is what the kernel takes")
                mixer["right"] = b
            else:
                problems.append(f"{where}type: {kind!r} is neither 'mamba1' nor 'parallel'")
                continue
            mlp = entry.get("mlp")
            if mlp is not None:
                lw = where + "mlp."
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    problems.append(f"{lw}kind: only 'dense' is built, config.json has {mlp!r}")
                    mlp = None
                else:
                    mlp = {"kind": "dense", "ff": positive_int(lw, mlp, "ff")}
            layers.append(ZodiraxLayer(kind, mixer, mlp))
        if problems:
            raise ConfigError("config.json cannot describe a Zodirax model:\n    "
                              + "\n    ".join(problems))
        return cls(vocab=vocab, width=width, eps=float(eps), embed_scale=embed_scale,
                   layers=tuple(layers),
                   initializer_range=float(raw.get("initializer_range", 0.05)))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""

        def pruned(v):
            if isinstance(v, dict):
                return {k: pruned(x) for k, x in v.items() if x is not None}
            return v

        layers = [{"type": layer.type, "mixer": pruned(layer.mixer), "mlp": layer.mlp}
                  for layer in self.layers]
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embed_scale},
                "layers": layers, "initializer_range": self.initializer_range}

    def model_spec(self) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.eps, suffix="", offset=NORM_OFFSET)
        blocks, ignore = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "mamba1":
                mixer = SelectiveScanSpec(hidden=self.width, inner=m["inner"], state=m["state"],
                                          dt_rank=m["dt_rank"], taps=m["conv"])
            else:
                a, b = m["left"], m["right"]
                position = None
                if a["rot"] is not None:
                    sc = a["rot"].get("scaling")
                    position = RotarySpec(
                        head_dim=a["dim"], rotary_dim=a["rot"]["dims"], theta=a["rot"]["base"],
                        max_positions=MAX_POSITIONS,
                        scaling=None if sc is None else BandScaling(
                            factor=sc["factor"], original=sc["original"], low=sc["low"],
                            high=sc["high"]))
                left = WindowSinkAttentionSpec(
                    hidden=self.width, heads=a["heads"], kv_heads=a["kv_heads"],
                    head_dim=a["dim"], value_dim=a["vdim"], scale=a["scale"],
                    window=None if a["mask"] is None else a["mask"]["size"],
                    keep_first=0 if a["mask"] is None else a["mask"]["keep_first"],
                    eps=self.eps, position=position, out_scale=m["left_scale"])
                right = DecayAttentionSpec(
                    hidden=self.width, heads=b["heads"], head_dim=b["dim"], value_dim=b["vdim"],
                    decay=tuple(b["decay"]), eps=self.eps, out_scale=m["right_scale"])
                mixer = ParallelMixerSpec(hidden=self.width, left=left, right=right)
            ffn = None
            if layer.mlp is not None:
                ffn = GatedMLPSpec(hidden=self.width, intermediate=layer.mlp["ff"],
                                   activation="silu", names=("gate", "up", "down"))
            else:      # a checkpoint may still carry the absent sublayer's norm
                ignore.append(f"l{i}.norm2")
            blocks.append(OutputNormBlockSpec(prefix=f"l{i}.", mixer=mixer, ffn=ffn, norm=norm))
        order = tuple(LayerCall(block=i, cache=i) for i in range(len(blocks)))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width,
            blocks=tuple(blocks), run_order=order, final_norm=norm, tie_head=True,
            max_positions=MAX_POSITIONS, embed_name="embed", final_norm_name="final.norm",
            stored_dtype="bfloat16", init_std=self.initializer_range,
            embed_scale=self.embed_scale, ignore_tensors=tuple(ignore))


register_architecture(ZodiraxConfig.architecture, ZodiraxConfig)
