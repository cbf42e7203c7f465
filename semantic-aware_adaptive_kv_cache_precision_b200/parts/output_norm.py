"""A layer whose norms sit on its sublayers' OUTPUTS only (`OutputNormBlockSpec`):

    x += norm1(mixer(x));   x += norm2(ffn(x))

on the fp32 residual stream; the sublayers read the stream itself. Between two sublayers ONE
pass over the stream norms the output of the one, adds it, and leaves the completed stream in
the type the next one reads (`RMSNorm.update`). What the layer's last sublayer produced leaves
the block as `pending` (a `NormedUpdate`), so that the next layer's first read does that pass.
Mixers and feed-forwards give their output through `produce(...)` (fp32 [T, hidden]); a part
that only has `forward(..., residual)` is given a zeroed tensor to add into.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, build_part, register_part
from .sandwich import NormedUpdate, _run


class OutputNormBlock(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        p = spec.prefix
        after_mixer, after_ffn = spec.norm_names
        self.mixer = build_part(spec.mixer, p + spec.mixer_name + ".", mode)
        self.mixer_after = build_part(spec.norm, p + after_mixer, mode)
        self.ffn = self.ffn_after = None
        if spec.ffn is not None:
            self.ffn = build_part(spec.ffn, p + spec.ffn_name + ".", mode)
            self.ffn_after = build_part(spec.norm, p + after_ffn, mode)
        self.parts = tuple(x for x in (self.mixer, self.mixer_after, self.ffn, self.ffn_after)
                           if x is not None)
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)
        self.kernel_libraries = ("norm_update",) + tuple(
            n for part in self.parts for n in getattr(part, "kernel_libraries", ()))

    def tensor_decls(self):
        return [d for part in self.parts for d in part.tensor_decls()]

    def bind(self, arena):
        for part in self.parts:
            part.bind(arena)

    def prepare(self, device, max_positions):
        for part in self.parts:
            part.prepare(device, max_positions)

    def cache_need(self):
        return self.mixer.cache_need()

    carries_pending = True

    def _stream(self, x, update=None):
        """The stream as the next sublayer reads it, after it has taken up `update`."""
        same = self.act_dtype == torch.float32          # the sublayer reads the stream itself
        if isinstance(update, NormedUpdate) and getattr(update.norm, "folds_update", False):
            h = update.norm.update(x, update.y, out_dtype=None if same else self.act_dtype)
            return x if same else h
        if update is not None:
            if hasattr(update, "apply"):
                update.apply(x)
            else:
                ops.add_into(x, update)
        return x if same else ops.rms_update(x, out_dtype=self.act_dtype)

    def forward(self, x, step, view, write_cache=True, pending=None, leave_pending=True):
        h = self._stream(x, pending)
        update = NormedUpdate(_run(self.mixer, h, step, view, write_cache), self.mixer_after)
        if self.ffn is not None:
            h = self._stream(x, update)
            update = NormedUpdate(_run(self.ffn, h, step), self.ffn_after)
        if leave_pending:
            return update
        update.apply(x)
        return None


register_part("output_norm_block", OutputNormBlock)
