"""The selective-scan mixer (`SelectiveScanSpec`):

    [x | z] = h Win^T
    x <- silu(conv(x) + b)           a causal convolution a channel over `taps` tokens
    [low | B | C] = x Wx^T;  dt = softplus(low Wdt^T + bdt);  A = -exp(A_log)
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c
    out = Wo [ y * silu(z) ]

Both projections that feed the recurrence leave fp32 (their accumulators, unrounded); the step
sizes (a product in fp32 and softplus), the decays and their exponentials, the state, the sums
over it and the gate are fp32 in both modes (`csrc/recurrent_scan.cu`). A sequence's state (S,
and the convolution's last `taps - 1` inputs) lives in the cache as two fixed-size states.

In bfloat16 a long part of a prompt is walked in runs of `RUN` tokens side by side. A step of
one token a sequence runs the convolution with its state update in one launch, and the scan's
kernel makes the step sizes itself.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import MultiNeed, StateNeed
from ..weights.decl import TensorDecl
from .base import Part, register_part


#: tokens a run when a long prompt is walked in runs side by side
RUN = 64


class SelectiveScanMixer(Part):
    kernel_libraries = ("recurrent_scan", "gemm_f32", "gemm_tc")

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.state > 512 or not 1 <= spec.taps <= 64:
            raise ValueError("the scan kernels take up to 512 states a channel and 1 to 64 taps")

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        return [TensorDecl(p + "in", (2 * s.inner, s.hidden)),
                TensorDecl(p + "conv", (s.inner, s.taps)),
                TensorDecl(p + "conv.b", (s.inner,)),
                TensorDecl(p + "x", (s.dt_rank + 2 * s.state, s.inner)),
                TensorDecl(p + "dt", (s.inner, s.dt_rank)),
                TensorDecl(p + "dt.b", (s.inner,), init="uniform", span=(-4.0, -1.0)),
                TensorDecl(p + "A_log", (s.inner, s.state), init="uniform", span=(-3.0, 1.0)),
                TensorDecl(p + "D", (s.inner,), init="ones_normal"),
                TensorDecl(p + "o", (s.hidden, s.inner))]

    def bind(self, arena):
        p = self.prefix
        self.w_in, self.w_x, self.w_o = (arena.view(p + n) for n in ("in", "x", "o"))
        self.conv_w, self.conv_b = arena.view(p + "conv"), arena.view(p + "conv.b")
        self.w_dt, self.b_dt = arena.view(p + "dt"), arena.view(p + "dt.b")
        self.a_log, self.d_skip = arena.view(p + "A_log"), arena.view(p + "D")

    def _run(self, step) -> int:
        """Tokens a run of a long prompt: in bfloat16 a sequence's part of the step is walked
        in runs side by side (the states carried between them in fp32). In the 32-bit mode,
        and for short parts, one walk, whose sums do not depend on how the sequence was cut."""
        if self.act_dtype == torch.float32 or getattr(step, "max_new", 0) < 4 * RUN:
            return 0
        return RUN

    def cache_need(self):
        s = self.spec
        return MultiNeed((StateNeed((s.taps - 1, s.inner), "float32"),
                          StateNeed((s.inner, s.state), "float32")))

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        s = self.spec
        conv_view, scan_view = view.parts
        xz = ops.linear(h, self.w_in, out_dtype=torch.float32)
        x = ops.causal_conv(xz, s.inner, self.conv_w, self.conv_b, conv_view.state, step,
                            self.act_dtype, keep_state=write_cache)
        low = ops.linear(x, self.w_x, out_dtype=torch.float32)
        # a step of one token a sequence makes its step sizes inside the scan's kernel
        dt = None if step.is_decode else ops.step_size(low, s.dt_rank, self.w_dt, self.b_dt)
        y = ops.selective_scan(x, dt, low, s.dt_rank, s.dt_rank + s.state, s.state,
                               xz[:, s.inner:], self.a_log, self.d_skip, scan_view.state, step,
                               keep_state=write_cache, run=self._run(step),
                               dt_weight=self.w_dt, dt_bias=self.b_dt)
        return ops.linear(y, self.w_o, out_dtype=torch.float32)

    def forward(self, h, step, view, residual, write_cache=True):
        ops.add_into(residual, self.produce(h, step, view, write_cache))


register_part("selective_scan", SelectiveScanMixer)
