"""Dense gated feed-forward: `residual += down( silu(gate(h)) * up(h) )`
(`src/microinfer/model.py:392-396`, `src/core_kernels/swiglu.cu:26-38`). Gate and
up are one product over the rows [Wgate; Wup] laid back to back in device
memory; the activation is fp32 inside with one rounding at its store."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.decl import TensorDecl
from .base import Part, register_part


class GatedMLP(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r}: only 'silu' is built")
        if spec.bias:
            raise ValueError("a gated feed-forward with biases is not built")

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        gate, up, down = self._names()
        return [TensorDecl(p + gate, (s.intermediate, s.hidden), group=p + "gate_up"),
                TensorDecl(p + up, (s.intermediate, s.hidden), group=p + "gate_up"),
                TensorDecl(p + down, (s.hidden, s.intermediate))]

    def _names(self):
        return getattr(self.spec, "names",
                       ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))

    def bind(self, arena):
        p = self.prefix
        gate, up, down = self._names()
        self.w_gate_up = arena.group_view(p + "gate_up")
        if self.w_gate_up is None:
            self.w_gate_up = torch.cat([arena.view(p + gate), arena.view(p + up)])
        self.w_down = arena.view(p + down)

    def produce(self, h, step):
        """The feed-forward's output as a tensor of its own, fp32 [T, hidden]."""
        return ops.linear(ops.gated_up(h, self.w_gate_up), self.w_down, out_dtype=torch.float32)

    can_defer = True

    def forward(self, h, step, residual, defer=False):
        act = ops.gated_up(h, self.w_gate_up)
        out = ops.linear(act, self.w_down, accumulate_into=residual, may_defer=defer)
        return out.delta if isinstance(out, ops.Deferred) else None


class DenseMLP(Part):
    """Dense feed-forward without a gate, `down(act(up(h)))`, with the tanh form of GELU
    (fp32 inside, one rounding at its store); tensors `up` and `down`."""

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.activation != "gelu_tanh":
            raise ValueError(f"activation {spec.activation!r}: only 'gelu_tanh' is built")

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        return [TensorDecl(p + "up", (s.intermediate, s.hidden)),
                TensorDecl(p + "down", (s.hidden, s.intermediate))]

    def bind(self, arena):
        self.w_up = arena.view(self.prefix + "up")
        self.w_down = arena.view(self.prefix + "down")

    def produce(self, h, step):
        """The feed-forward's output, fp32 [T, hidden]."""
        act = ops.gelu_tanh(ops.linear(h, self.w_up, out_dtype=self.act_dtype))
        return ops.linear(act, self.w_down, out_dtype=torch.float32)

    def forward(self, h, step, residual):
        ops.linear(ops.gelu_tanh(ops.linear(h, self.w_up, out_dtype=self.act_dtype)),
                   self.w_down, accumulate_into=residual)


register_part("gated_mlp", GatedMLP)
register_part("dense_mlp", DenseMLP)
