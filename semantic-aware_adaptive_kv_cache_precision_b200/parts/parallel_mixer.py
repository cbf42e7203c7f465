"""Two mixers side by side that read the same input (`ParallelMixerSpec`); the mixer's output
is the sum of theirs, each multiplied by its own `out_scale` on its way:

    out = Wo_a [mix_a(h)] + Wo_b [mix_b(h)]

Every matrix of both branches that reads the mixer's input is laid back to back in the arena,
so the step runs ONE product for all of them (its fp32 result is cut by column offsets), then
each branch's own kernels, then the two output products, the second adding into the first.

A branch is any part with the branch interface: `input_rows`, `input_decls(group)`,
`other_decls()`, `input_bias(arena)`, `bind_rest(arena)`, `mix(proj, offset, h, step, view,
write_cache)`, `w_o`, `cache_need()`.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import MultiNeed
from .base import Part, build_part, register_part


class ParallelMixer(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        self.branches = tuple(build_part(b, f"{prefix}{name}.", mode)
                              for b, name in zip((spec.left, spec.right), spec.names))
        for b in self.branches:
            if not hasattr(b, "mix"):
                raise TypeError(f"{type(b).__name__} cannot stand beside another mixer: it has "
                                "no `mix`")
        self.graph_safe = all(getattr(b, "graph_safe", True) for b in self.branches)
        self.kernel_libraries = tuple(n for b in self.branches
                                      for n in getattr(b, "kernel_libraries", ()))
        self.offsets, at = [], 0
        for b in self.branches:
            self.offsets.append(at)
            at += b.input_rows
        self.rows = at

    def tensor_decls(self):
        group = self.prefix + "fused"
        decls = [d for b in self.branches for d in b.input_decls(group)]
        return decls + [d for b in self.branches for d in b.other_decls()]

    def bind(self, arena):
        self.w_in = arena.group_view(self.prefix + "fused")
        if self.w_in is None:
            self.w_in = torch.cat([arena.view(d.name) for b in self.branches
                                   for d in b.input_decls(None)])
        biases = [b.input_bias(arena) for b in self.branches]
        self.b_in = None
        if any(x is not None for x in biases):      # zeros complete the vector
            some = next(x for x in biases if x is not None)
            self.b_in = torch.cat([x if x is not None else
                                   torch.zeros(b.input_rows, dtype=some.dtype, device=some.device)
                                   for b, x in zip(self.branches, biases)])
        for b in self.branches:
            b.bind_rest(arena)

    def prepare(self, device, max_positions):
        for b in self.branches:
            b.prepare(device, max_positions)

    def cache_need(self):
        return MultiNeed(tuple(b.cache_need() for b in self.branches))

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        proj = ops.linear(h, self.w_in, self.b_in, out_dtype=torch.float32)
        out = None
        for b, offset, part in zip(self.branches, self.offsets, view.parts):
            mixed = b.mix(proj, offset, h, step, part, write_cache)
            if out is None:
                out = ops.linear(mixed, b.w_o, out_dtype=torch.float32)
            else:
                ops.linear(mixed, b.w_o, accumulate_into=out)
        return out

    def forward(self, h, step, view, residual, write_cache=True):
        ops.add_into(residual, self.produce(h, step, view, write_cache))


register_part("parallel_mixer", ParallelMixer)
