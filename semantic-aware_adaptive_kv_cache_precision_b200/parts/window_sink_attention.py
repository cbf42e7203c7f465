"""Grouped-query attention over a window that keeps a sequence's first tokens, with a learned
logit a head in the softmax's denominator (`WindowSinkAttentionSpec`):

    [q | k | v] = h Wfused^T + b
    q <- q / rms(q) * wq,  k <- k / rms(k) * wk      (over the WHOLE projection, all heads at once)
    the first `rotary_dim` numbers of every head of q and k turned by the position
    s_ij = q_i . k_j * scale  for  j <= i  and  (i - j < window  or  j < keep_first)
    a_i = sum_j exp(s_ij) v_j / (sum_j exp(s_ij) + exp(sink[h]))
    out = Wo [out_scale * a]

The fused projection leaves fp32 (its accumulator, unrounded); the two norms, the rotation and
the cache write are one kernel (`csrc/qk_prepare.cu`); scores, softmax weights, the sink and the
weighted sums are fp32 in both modes (`csrc/attention_distance.cu`). The cache keeps the blocks
of the first `keep_first` positions for as long as the sequence lives (`KVNeed.keep_first`).

The part is a mixer of its own (`produce`) and a branch of a `ParallelMixer` (`input_rows`,
`input_decls`, `input_bias`, `mix`, `w_o`).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import KVNeed
from ..weights.decl import TensorDecl
from .base import Part, build_part, register_part


class WindowSinkAttention(Part):
    kernel_libraries = ("qk_prepare", "attention_distance", "gemm_f32", "gemm_tc")

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"{s.heads} heads are not a multiple of {s.kv_heads} kv heads")
        if s.head_dim > 640 or s.value_dim > 512:
            raise ValueError("the attention kernel takes head_dim up to 640 and value_dim up to 512")
        if s.qk_norm not in (None, "whole"):
            raise ValueError(f"qk_norm {s.qk_norm!r}: only 'whole' (or None) is built")
        if s.keep_first and not s.window:
            raise ValueError("keep_first goes with a window")
        self.q_cols = s.heads * s.head_dim
        self.k_cols = s.kv_heads * s.head_dim
        self.v_cols = s.kv_heads * s.value_dim
        self.position = None if s.position is None else build_part(s.position, prefix, mode)
        self.sink = None

    # -- what a branch offers -------------------------------------------------------------

    @property
    def input_rows(self) -> int:
        return self.q_cols + self.k_cols + self.v_cols

    def _inputs(self):
        return (("q", self.q_cols), ("k", self.k_cols), ("v", self.v_cols))

    def input_decls(self, group):
        """The matrices that read the mixer's input, in the order of their rows in the fused
        product, laid back to back under `group`."""
        s, p = self.spec, self.prefix
        return [TensorDecl(p + n, (rows, s.hidden), group=group) for n, rows in self._inputs()]

    def other_decls(self):
        s, p = self.spec, self.prefix
        decls = []
        if s.bias:
            decls += [TensorDecl(f"{p}{n}.b", (rows,), group=p + "fused.b")
                      for n, rows in self._inputs()]
        if s.qk_norm:
            decls += [TensorDecl(p + "q.norm", (self.q_cols,), init="ones_normal"),
                      TensorDecl(p + "k.norm", (self.k_cols,), init="ones_normal")]
        if s.sink:
            decls.append(TensorDecl(p + "sink", (s.heads,)))
        decls.append(TensorDecl(p + "o", (s.hidden, s.heads * s.value_dim)))
        return decls

    def input_bias(self, arena):
        """The fused product's bias [input_rows], or None."""
        if not self.spec.bias:
            return None
        p = self.prefix
        b = arena.group_view(p + "fused.b")
        if b is None:
            b = torch.cat([arena.view(f"{p}{n}.b") for n, _ in self._inputs()])
        return b

    def bind_rest(self, arena):
        s, p = self.spec, self.prefix
        self.wq = arena.view(p + "q.norm") if s.qk_norm else None
        self.wk = arena.view(p + "k.norm") if s.qk_norm else None
        self.sink = arena.view(p + "sink").float().contiguous() if s.sink else None
        self.w_o = arena.view(p + "o")

    def mix(self, proj, offset, h, step, view, write_cache=True):
        """From the fused product `proj` (fp32 [T, columns], this branch's columns from
        `offset` on) to the input of `w_o`: [T, heads * value_dim] of the activations' type,
        `out_scale` included."""
        s = self.spec
        cos = sin = None
        if self.position is not None:
            if step.max_position >= self.position.cos.shape[0]:
                raise ValueError(f"position {step.max_position} is beyond the rotary table of "
                                 f"{self.position.cos.shape[0]} positions")
            cos, sin = self.position.cos, self.position.sin
        q = ops.qk_prepare(proj, offset, offset + self.q_cols, offset + self.q_cols + self.k_cols,
                           s.heads, s.kv_heads, s.head_dim, s.value_dim, self.wq, self.wk, s.eps,
                           cos, sin, step.positions, step.token_seq, view.block_table, view.keys,
                           view.values, self.act_dtype, write_cache)
        return ops.cached_attention(
            q.view(q.shape[0], s.heads, s.head_dim), view.keys, view.values, step.positions,
            step.token_seq, view.block_table, s.heads, s.head_dim, s.value_dim, s.scale,
            window=s.window, keep_first=s.keep_first if s.window else 0, sink=self.sink,
            out_scale=s.out_scale, **self._decode_form(step)).view(q.shape[0], -1)

    def _decode_form(self, step) -> dict:
        """For decode steps in bfloat16 a block's warps are one token's groups of heads and
        share each chunk of its keys; several blocks a token take shares of the chunks. In the
        32-bit mode and for prompts a warp walks its token's keys alone, in the order of their
        positions, so the sums do not depend on how the prompt was cut."""
        if self.act_dtype == torch.float32 or not step.is_decode:
            return {}
        s = self.spec
        keys = step.max_len_bound or step.max_len
        if s.window:
            keys = min(keys, s.window + s.keep_first + 63)
        return {"heads_first": True,
                "key_splits": ops.plan_token_blocks(keys, step.tokens * s.kv_heads)}

    # -- the part alone ---------------------------------------------------------------------

    def tensor_decls(self):
        return self.input_decls(self.prefix + "fused") + self.other_decls()

    def bind(self, arena):
        p = self.prefix
        self.w_in = arena.group_view(p + "fused")
        if self.w_in is None:
            self.w_in = torch.cat([arena.view(p + n) for n, _ in self._inputs()])
        self.b_in = self.input_bias(arena)
        self.bind_rest(arena)

    def prepare(self, device, max_positions):
        if self.position is not None:
            self.position.prepare(device, max_positions)

    def cache_need(self):
        s = self.spec
        return KVNeed(s.kv_heads, s.head_dim, s.window, value_dim=s.value_dim,
                      keep_first=s.keep_first if s.window else 0)

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        proj = ops.linear(h, self.w_in, self.b_in, out_dtype=torch.float32)
        return ops.linear(self.mix(proj, 0, h, step, view, write_cache), self.w_o,
                          out_dtype=torch.float32)

    def forward(self, h, step, view, residual, write_cache=True):
        proj = ops.linear(h, self.w_in, self.b_in, out_dtype=torch.float32)
        ops.linear(self.mix(proj, 0, h, step, view, write_cache), self.w_o,
                   accumulate_into=residual)


register_part("window_sink_attention", WindowSinkAttention)
