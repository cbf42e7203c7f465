"""Causal attention over one cached latent a position (`LatentAttentionSpec`).

    [cq | ckv | kr] = h Wdown^T;  cq = rms(cq) wq;  c = rms(ckv) wkv;  kr = rotate(kr)
    cache <- [c | kr]                                  (kv_rank + rot_dim numbers a position)
    q_h = [qp_h | rotate(qr_h)] = cq Wuq_h^T           (head_dim plain, rot_dim rotated)
    s_ij = (qp_h . Wuk_h c_j + qr_h . kr_j) * scale;   out_h = Wuv_h sum_j softmax(s)_ij c_j

With a `window` w the sum runs over 0 <= i - j < w only (and the cache gives back the blocks
behind it); with `sink` the softmax's denominator of head h also holds exp(sink_h); with
`head_gate` out_h is multiplied by sigmoid(Wg h)_h, whose rows lie behind the query's in one
product. The rotation pairs halves or neighbours, as the position part says.

The keys and values of a head are never made: since `qp_h . (Wuk_h c) = (Wuk_h^T qp_h) . c`,
each head's plain query is carried into the latent's space (a batched product over the heads),
attention runs with one shared key row [c | kr] a position for all heads and returns weighted
sums of latents, and a second batched product takes those to the heads' values. Norms,
rotation angles, scores, softmax weights and the weighted sums are fp32 in both modes
(`csrc/latent.cu`, `csrc/attention_distance.cu`).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import KVNeed
from ..weights.decl import TensorDecl
from .base import Part, build_part, register_part


class LatentAttention(Part):
    kernel_libraries = ("latent", "attention_distance", "gemm_f32", "gemm_tc")

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        s = spec
        if s.position.rotary_dim != s.rot_dim or s.rot_dim % 2:
            raise ValueError(f"the rotation's {s.position.rotary_dim} dimensions must be the "
                             f"mixer's rot_dim {s.rot_dim}, an even number")
        if s.kv_rank + s.rot_dim > 640 or s.kv_rank > 512:
            raise ValueError("the attention kernel takes kv_rank + rot_dim up to 640 and "
                             "kv_rank up to 512")
        self.position = build_part(s.position, prefix, mode)
        self.q_width = s.head_dim + s.rot_dim

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        down = []
        if s.q_rank:
            down.append(TensorDecl(p + "dq", (s.q_rank, s.hidden), group=p + "down"))
        down.append(TensorDecl(p + "dkv", (s.kv_rank + s.rot_dim, s.hidden), group=p + "down"))
        decls = down
        if s.q_rank:
            decls += [TensorDecl(p + "dq.norm", (s.q_rank,), init="ones_normal"),
                      TensorDecl(p + "uq", (s.heads * self.q_width, s.q_rank))]
        else:
            decls.append(TensorDecl(p + "q", (s.heads * self.q_width, s.hidden), group=p + "up"))
        if s.head_gate:            # behind the queries' rows: one product makes both
            decls.append(TensorDecl(p + "g", (s.heads, s.q_rank or s.hidden),
                                    group=None if s.q_rank else p + "up"))
        if s.sink:
            decls.append(TensorDecl(p + "sink", (s.heads,)))
        decls += [TensorDecl(p + "dkv.norm", (s.kv_rank,), init="ones_normal"),
                  TensorDecl(p + "uk", (s.heads * s.head_dim, s.kv_rank)),
                  TensorDecl(p + "uv", (s.heads * s.value_dim, s.kv_rank)),
                  TensorDecl(p + "o", (s.hidden, s.heads * s.value_dim))]
        return decls

    def bind(self, arena):
        s, p = self.spec, self.prefix
        self.w_down = arena.group_view(p + "down")
        if self.w_down is None:
            self.w_down = torch.cat([arena.view(p + n) for n in (("dq", "dkv") if s.q_rank
                                                                 else ("dkv",))])
        # (the small tensors below take the activations' type whatever the checkpoint's)
        self.q_norm = arena.view(p + "dq.norm").to(self.act_dtype) if s.q_rank else None
        self.w_q = arena.view(p + ("uq" if s.q_rank else "q"))
        self.w_gate = None
        if s.head_gate:
            if s.q_rank:
                raise ValueError("a gate a head beside a query latent is not built")
            both = arena.group_view(p + "up")
            if both is None:
                both = torch.cat([self.w_q, arena.view(p + "g")])
            self.w_q = both        # [queries; gates]
        self.sink = arena.view(p + "sink").float().contiguous() if s.sink else None
        self.kv_norm = arena.view(p + "dkv.norm").to(self.act_dtype)
        # [heads, kv_rank, head_dim]: the rows of Wuk_h^T, which carry a plain query to the
        # latent's space (a small copy, made once)
        self.w_uk_t = arena.view(p + "uk").view(s.heads, s.head_dim, s.kv_rank) \
            .transpose(1, 2).to(self.act_dtype).contiguous()
        self.w_uv = arena.view(p + "uv").view(s.heads, s.value_dim, s.kv_rank).to(self.act_dtype)
        self.w_o = arena.view(p + "o")

    def prepare(self, device, max_positions):
        self.position.prepare(device, max_positions)

    def cache_need(self):
        s = self.spec
        return KVNeed(1, s.kv_rank + s.rot_dim, s.window, value_dim=0)

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        return ops.linear(self._heads(h, step, view, write_cache), self.w_o,
                          out_dtype=torch.float32)

    def _heads(self, h, step, view, write_cache):
        """The heads' outputs side by side, [T, heads * value_dim]: the input of `w_o`."""
        s, pos = self.spec, self.position
        if step.max_position >= pos.cos.shape[0]:
            raise ValueError(f"position {step.max_position} is beyond the rotary table of "
                             f"{pos.cos.shape[0]} positions")
        tokens, rank = h.shape[0], s.kv_rank
        q_rank = s.q_rank or 0
        down = ops.linear(h, self.w_down, out_dtype=torch.float32)
        q_latent = ops.latent_prepare(down, q_rank, rank, s.rot_dim, self.q_norm, self.kv_norm,
                                      s.eps, step, view, pos.cos, pos.sin, self.act_dtype,
                                      write_cache, pos.interleaved)
        q = ops.linear(q_latent if s.q_rank else h, self.w_q, out_dtype=self.act_dtype)
        ops.rotate_heads(q, self.q_width, s.head_dim, s.heads, s.rot_dim, step.positions,
                         pos.cos, pos.sin, pos.interleaved)
        q_cols = s.heads * self.q_width
        q3 = q[:, :q_cols].view(tokens, s.heads, self.q_width)
        # every head's plain query in the latent's space
        in_latent = torch.empty((tokens, s.heads, rank), dtype=q.dtype, device=q.device)
        ops.per_head(q3[:, :, :s.head_dim], self.w_uk_t, in_latent)
        mixed = ops.cached_attention(
            in_latent, view.keys, None, step.positions, step.token_seq, view.block_table,
            s.heads, rank + s.rot_dim, rank, s.scale, q2=q3[:, :, s.head_dim:], q_split=rank,
            window=s.window, sink=self.sink,
            head_gate=q[:, q_cols:] if s.head_gate else None, **self._decode_form(step, q))
        # the weighted sums of latents to each head's values
        heads_out = torch.empty((tokens, s.heads, s.value_dim), dtype=q.dtype, device=q.device)
        ops.per_head(mixed.view(tokens, s.heads, rank), self.w_uv, heads_out)
        return heads_out.view(tokens, s.heads * s.value_dim)

    def _decode_form(self, step, q) -> dict:
        """How a step's tokens share their keys. Prompts, and everything in the 32-bit mode:
        a warp a token and group of heads walks the keys alone (the sums then have one order
        however the tokens are cut). Decode steps in bfloat16: a block's warps are one token's
        groups of heads and share each chunk of rows through shared memory, and several blocks
        a token take shares of the chunks, as many as `ops.plan_token_blocks` gives for the
        longest sequence the step's block lists can hold (a captured step keeps its launch
        numbers as long as they do)."""
        if q.dtype == torch.float32 or not step.is_decode:
            return {}
        keys = step.max_len_bound or step.max_len
        if self.spec.window:         # (a window's first chunk and its last may both be partial)
            keys = min(keys, self.spec.window + 63)
        return {"heads_first": True, "key_splits": ops.plan_token_blocks(keys, step.tokens)}

    def forward(self, h, step, view, residual, write_cache=True):
        ops.linear(self._heads(h, step, view, write_cache), self.w_o, accumulate_into=residual)


register_part("latent_attention", LatentAttention)
