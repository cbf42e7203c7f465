"""A mixture of clamped gated feed-forwards with a shared one (`RoutedExpertsSpec`):

    z = h Wrouter^T (fp32);  s = sigmoid(z), or softmax(z) over all the router's outputs
    the `top` largest s (+ a learned correction an output, for the choice only) choose a
    token's experts; the last `identity` outputs stand for experts that return their input
    expert_e(x) = Wdown_e [ g * sigmoid(alpha g) * (u + 1) ],  g = min(Wgate_e x, limit),
                                                              u = clamp(Wup_e x, -limit, limit)
    out = sum_chosen expert_e(s_e h)  +  sigmoid(h Wsg^T) * shared(h)

The chosen scores are used as they are (or divided by their sum with `renormalize`) and
multiply the expert's INPUT (`weight_input`) or its output. Everything stays on the device:
the router's product runs in fp32 on the step's tokens, a kernel chooses and counts, the
tokens' rows are sorted by expert, and two grouped products (gate and up with the activation
in the epilogue, then down) run over tiles of one expert's rows each (`csrc/moe.cu`). The
experts' matrices lie back to back in the arena, so a tile finds its expert's weights by
index. The shared expert is a dense feed-forward of the same form on the usual products.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import mixture
from ..weights.decl import TensorDecl
from .base import Part, register_part


class RoutedExperts(Part):
    kernel_libraries = ("moe", "gemm_f32", "gemm_tc")

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.score not in ("sigmoid", "softmax"):
            raise ValueError(f"router score {spec.score!r}: 'sigmoid' and 'softmax' are built")
        if spec.renormalize:
            raise ValueError("renormalized router weights are not built")
        self.outputs = spec.experts + spec.identity
        if spec.experts < 1 or spec.identity < 0 or spec.top > self.outputs \
                or self.outputs > 1024 or spec.top > 32:
            raise ValueError("the router takes up to 1024 outputs (experts and identity "
                             "experts) and top up to 32 of them")

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        ff = s.expert.intermediate
        decls = []
        for name, shape in (("gate", (ff, s.hidden)), ("up", (ff, s.hidden)),
                            ("down", (s.hidden, ff))):
            decls += [TensorDecl(f"{p}e{e}.{name}", shape, group=f"{p}experts.{name}")
                      for e in range(s.experts)]
        decls.append(TensorDecl(p + "router", (self.outputs, s.hidden), group=p + "route"))
        if s.correction:
            decls.append(TensorDecl(p + "correction", (self.outputs,)))
        if s.shared is not None:
            fs = s.shared.intermediate
            if s.shared_gate:
                decls.append(TensorDecl(p + "shared.sg", (1, s.hidden), group=p + "route"))
            decls += [TensorDecl(p + "shared.gate", (fs, s.hidden), group=p + "shared.gate_up"),
                      TensorDecl(p + "shared.up", (fs, s.hidden), group=p + "shared.gate_up"),
                      TensorDecl(p + "shared.down", (s.hidden, fs))]
        return decls

    def bind(self, arena):
        s, p = self.spec, self.prefix
        ff = s.expert.intermediate

        def stacked(name, rows, cols):
            w = arena.group_view(f"{p}experts.{name}")
            if w is None:
                w = torch.cat([arena.view(f"{p}e{e}.{name}") for e in range(s.experts)])
            return w.view(s.experts, rows, cols)

        self.w_gate = stacked("gate", ff, s.hidden)
        self.w_up = stacked("up", ff, s.hidden)
        self.w_down = stacked("down", s.hidden, ff)
        route = [arena.view(p + "router")]
        self.has_gate = s.shared is not None and s.shared_gate
        if self.has_gate:
            route.append(arena.view(p + "shared.sg"))
        # the router's product is 32-bit in both modes: its rows are kept widened
        self.w_route = torch.cat(route).float().contiguous()
        self.correction = arena.view(p + "correction").float().contiguous() if s.correction \
            else None
        if s.shared is not None:
            self.w_shared_in = arena.group_view(p + "shared.gate_up")
            if self.w_shared_in is None:
                self.w_shared_in = torch.cat([arena.view(p + "shared.gate"),
                                              arena.view(p + "shared.up")])
            self.w_shared_down = arena.view(p + "shared.down")

    def produce(self, h, step, into=None):
        """The feed-forward's output, fp32 [T, hidden]; with `into` (the fp32 stream) it is
        added there by the kernel that sums a token's rows."""
        s = self.spec
        logits = mixture.router_logits(h, self.w_route)
        routing = mixture.route(logits, s.experts, s.top, s.identity, s.score == "softmax",
                                self.correction)
        # (a checkpoint stored in 32 bits keeps its matrices so: the experts then run in 32 bits)
        rows = mixture.gather_rows(h if h.dtype == self.w_gate.dtype else h.to(self.w_gate.dtype),
                                   routing, s.weight_input)
        act = mixture.grouped_product(rows, routing, self.w_gate, self.w_up, s.expert.limit,
                                      s.expert.alpha)
        products = mixture.grouped_product(act, routing, self.w_down, None)
        shared = gate = None
        if s.shared is not None:
            both = ops.linear(h, self.w_shared_in, out_dtype=self.act_dtype)
            shared = ops.linear(mixture.clamped_act(both, s.shared.limit, s.shared.alpha),
                                self.w_shared_down, out_dtype=torch.float32)
            gate = logits[:, self.outputs] if self.has_gate else None
        return mixture.combine(products, routing, not s.weight_input, shared, gate, h, into)

    def forward(self, h, step, residual):
        self.produce(h, step, into=residual)


register_part("routed_experts", RoutedExperts)
