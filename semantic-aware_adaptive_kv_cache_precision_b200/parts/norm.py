"""RMSNorm: `x * rsqrt(mean(x^2) + eps) * w` over rows of the fp32 residual
stream (`src/core_kernels/rmsnorm.cu:33-84`; the weight multiplies directly). With
`NormSpec.offset` the multiplier is `offset + w` (weights stored around zero); such a norm
can also complete the stream with a sublayer's normed output on its way (`update`)."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.decl import TensorDecl
from .base import Part, register_part


class RMSNorm(Part):
    """`prefix` is the tensor's name without the spec's suffix ('.weight' by default)."""

    @property
    def weight_name(self):
        return self.prefix + getattr(self.spec, "suffix", ".weight")

    @property
    def offset(self) -> float:
        return float(getattr(self.spec, "offset", 0.0))

    def tensor_decls(self):
        return [TensorDecl(self.weight_name, (self.spec.size,),
                           init="normal" if self.offset else "ones_normal")]

    def bind(self, arena):
        self.weight = arena.view(self.weight_name)

    folds_add = True     # forward(x, add=delta) does x += delta on its way

    def forward(self, x, out_dtype=None, rows=None, add=None):
        out_dtype = out_dtype or self.act_dtype
        if self.offset:
            if add is not None:
                ops.add_into(x, add)
            return ops.rms_update(x, out_dtype=out_dtype, out_weight=self.weight,
                                  out_offset=self.offset, eps=self.spec.eps, rows=rows)
        if add is not None and (rows is not None or out_dtype != torch.bfloat16
                                or self.weight.dtype != torch.bfloat16):
            ops.add_into(x, add)
            add = None
        return ops.rms_norm(x, self.weight, self.spec.eps, out_dtype, rows, add)

    folds_update = True  # update(x, y, out_dtype) does x += norm(y) and hands the stream on

    def update(self, x, y, out_dtype=None):
        """`x += norm(y)` in place on the fp32 stream; with `out_dtype`, also returns the
        completed stream in that type (what a sublayer that reads the stream itself takes)."""
        return ops.rms_update(x, y, add_weight=self.weight, add_offset=self.offset,
                              out_dtype=out_dtype, eps=self.spec.eps)

    def complete(self, x, y):
        self.update(x, y)


class LayerNorm(RMSNorm):
    kernel_libraries = ("layer_norm", "elementwise")

    """`(x - mean) / sqrt(variance + eps) * w` over rows of the fp32 stream, no bias; the
    variance is the mean of the squared deviations (`csrc/layer_norm.cu`).

    `forward(x, add=y, add_norm=other)` first completes the stream with a sublayer's normed
    output, `x += other(y)`, in the same pass (`other`: the `LayerNorm` after that sublayer);
    `complete(x, y)` does only that."""

    folds_add = False            # a plain delta is added by `ops.add_into` first
    folds_normed = True
    folds_update = False

    def forward(self, x, out_dtype=None, rows=None, add=None, add_norm=None):
        out_dtype = out_dtype or self.act_dtype
        if add is not None and add_norm is None:
            ops.add_into(x, add)
            add = None
        if add is not None and (rows is not None or add_norm.spec.eps != self.spec.eps
                                or add_norm.weight.dtype != self.weight.dtype):
            add_norm.complete(x, add)
            add = None
        return ops.layer_norm(x, self.weight, self.spec.eps, out_dtype, rows, add,
                              None if add is None else add_norm.weight)

    def complete(self, x, y):
        """`x += norm(y)`, in place on the fp32 stream."""
        ops.layer_norm(x, None, self.spec.eps, torch.float32, add=y, add_weight=self.weight)


register_part("rms_norm", RMSNorm)
register_part("layer_norm", LayerNorm)
