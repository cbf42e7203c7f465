"""Attention without softmax over a state that fades by a fixed factor a head
(`DecayAttentionSpec`):

    [q | k | v | g] = h Wfused^T;   q, k, v <- silu(q), silu(k), silu(v)
    S <- decay[h] S + k v^T;   o = S^T q                        (a head; S is dim x value_dim)
    out = Wo [ o / rms(o) * w * sigmoid(g) * out_scale ]        (rms over ALL heads' outputs)

The fused projection leaves fp32 (its accumulator, unrounded); the silus, the recurrence, the
norm and the gate are fp32 in both modes (`csrc/recurrent_scan.cu`). The state lives in the
cache as fixed-size per-sequence state, stored as its transpose [heads, value_dim, dim]. The
state moves by its change, `S += (decay - 1) S + k v^T`, with `decay - 1` rounded once from the
exact number; in bfloat16 a long part of a prompt is walked in runs of `RUN` tokens side by side.

The spec's fields turn this into its relatives: no activation on q, k, v; the first numbers of
every head of q and k turned by the token's position (the tables of a `RotaryHalf`, rotation in
fp32 as the rows enter the recurrence); k multiplied by a constant after that; the root mean
square taken a head instead of over all heads, with or without a weight; `silu` instead of
`sigmoid` for the gate. With all of them: retention,

    q, k <- turn(q), turn(k) * dim^(-1/2);   o_h <- o_h / rms(o_h);   out = Wo [ o * silu(g) ]

The part is a mixer of its own (`produce`) and a branch of a `ParallelMixer`.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import StateNeed
from ..weights.decl import TensorDecl
from .base import Part, build_part, register_part


#: tokens a run when a long prompt is walked in runs side by side
RUN = 64


class DecayAttention(Part):
    kernel_libraries = ("recurrent_scan", "gemm_f32", "gemm_tc")

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        s = spec
        if s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim}: the recurrence kernel takes up to 256")
        if len(s.decay) != s.heads:
            raise ValueError(f"{len(s.decay)} decays for {s.heads} heads")
        if s.activation not in (None, "silu") or s.norm not in ("all", "head") \
                or s.gate_kind not in ("sigmoid", "silu"):
            raise ValueError(f"activation {s.activation!r}, norm {s.norm!r} or gate "
                             f"{s.gate_kind!r} is not built")
        self.position = None
        if s.position is not None:
            if s.position.kind != "rotary_half" or s.position.rotary_dim > s.head_dim:
                raise ValueError("the recurrence kernel turns pairs (i, i + dims / 2) of the "
                                 "first dims <= head_dim numbers of a head")
            self.position = build_part(s.position, prefix, mode)
        self.qk_cols = s.heads * s.head_dim
        self.v_cols = s.heads * s.value_dim
        self.decay_less_one = None

    # -- what a branch offers -------------------------------------------------------------

    def _inputs(self):
        rows = [("q", self.qk_cols), ("k", self.qk_cols), ("v", self.v_cols)]
        if self.spec.gate:
            rows.append(("g", self.v_cols))
        return tuple(rows)

    @property
    def input_rows(self) -> int:
        return sum(rows for _, rows in self._inputs())

    def input_decls(self, group):
        s, p = self.spec, self.prefix
        return [TensorDecl(p + n, (rows, s.hidden), group=group) for n, rows in self._inputs()]

    def other_decls(self):
        s, p = self.spec, self.prefix
        norm = [TensorDecl(p + "norm", (self.v_cols,), init="ones_normal")] if s.norm_weight else []
        return norm + [TensorDecl(p + "o", (s.hidden, self.v_cols))]

    def input_bias(self, arena):
        return None

    def bind_rest(self, arena):
        p = self.prefix
        self.norm_w = arena.view(p + "norm") if self.spec.norm_weight else None
        self.w_o = arena.view(p + "o")
        # the kernel takes `decay - 1`, rounded to fp32 once from the exact number
        self.decay_less_one = (torch.tensor(self.spec.decay, dtype=torch.float64) - 1.0).to(
            device=self.w_o.device, dtype=torch.float32)

    def mix(self, proj, offset, h, step, view, write_cache=True):
        """From the fused product `proj` (fp32 [T, columns], this branch's columns from
        `offset` on) to the input of `w_o`: [T, heads * value_dim] of the activations' type,
        `out_scale` included."""
        s = self.spec
        k_off, v_off = offset + self.qk_cols, offset + 2 * self.qk_cols
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.cos, self.position.sin
            if step.max_position >= cos.shape[0]:
                raise ValueError(f"position {step.max_position} is beyond the rotary table of "
                                 f"{cos.shape[0]} positions")
        y = ops.decay_attention(proj, offset, k_off, v_off, s.heads, s.head_dim, s.value_dim,
                                self.decay_less_one, view.state, step, keep_state=write_cache,
                                run=self._run(step), activation=s.activation == "silu",
                                cos=cos, sin=sin, key_scale=s.key_scale)
        gate = proj[:, v_off + self.v_cols:v_off + 2 * self.v_cols] if s.gate else None
        return ops.norm_gate(y, self.norm_w, gate, s.eps, s.out_scale, self.act_dtype,
                             group=s.value_dim if s.norm == "head" else None,
                             gate_silu=s.gate_kind == "silu")

    # -- the part alone ---------------------------------------------------------------------

    def tensor_decls(self):
        return self.input_decls(self.prefix + "fused") + self.other_decls()

    def bind(self, arena):
        p = self.prefix
        self.w_in = arena.group_view(p + "fused")
        if self.w_in is None:
            self.w_in = torch.cat([arena.view(p + n) for n, _ in self._inputs()])
        self.bind_rest(arena)

    def _run(self, step) -> int:
        """Tokens a run of a long prompt: in bfloat16 a sequence's part of the step is walked
        in runs side by side (the states carried between them in fp32). In the 32-bit mode,
        and for short parts, one walk, whose sums do not depend on how the sequence was cut."""
        if self.act_dtype == torch.float32 or getattr(step, "max_new", 0) < 4 * RUN:
            return 0
        return RUN

    def prepare(self, device, max_positions):
        if self.position is not None:
            self.position.prepare(device, max_positions)

    def cache_need(self):
        s = self.spec
        return StateNeed((s.heads, s.value_dim, s.head_dim), "float32")

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)
        return ops.linear(self.mix(proj, 0, h, step, view, write_cache), self.w_o,
                          out_dtype=torch.float32)

    def forward(self, h, step, view, residual, write_cache=True):
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)
        ops.linear(self.mix(proj, 0, h, step, view, write_cache), self.w_o,
                   accumulate_into=residual)


register_part("decay_attention", DecayAttention)
