"""Rotate-half rotary position encoding.

The table of cos and sin of `pos * theta^(-2j/rot)` is built on the host in
float64 and kept in fp32, as the reference builds it
(`src/core_kernels/rope_table.cu:18-31`, `rope_angle.cuh:15-21`); the kernel
rotates in fp32 (`csrc/rope.cu`). Queries are rotated in place; keys are rotated
on their way into the cache, in the same launch that stores the values.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import Part, register_part


class RotaryHalf(Part):
    #: which numbers of a head make a pair: False (i, i + rotary_dim / 2), True (2i, 2i + 1)
    interleaved = False

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and in "
                             f"(0, head_dim {spec.head_dim}]")
        self.cos = self.sin = None

    def prepare(self, device, max_positions):
        n = min(max_positions, self.spec.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n and self.cos.device == torch.device(device):
            return
        inv_freq, magnitude = self.frequencies()
        angle = np.arange(n, dtype=np.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.from_numpy((np.cos(angle) * magnitude).astype(np.float32)).to(device)
        self.sin = torch.from_numpy((np.sin(angle) * magnitude).astype(np.float32)).to(device)

    def frequencies(self):
        """(float64 [rotary_dim / 2], magnitude): pair i turns by `position * f_i`, f_i =
        theta^(-2i / rotary_dim). With `spec.scaling` the pairs whose wavelength is long
        against the original context turn `factor` times slower, the short ones as before,
        a linear ramp over the pair index between the two (from the index whose wavelength
        makes `fast` turns in `original` positions to the one that makes `slow`), and the
        table's cosines and sines are multiplied by `magnitude_slope * ln(factor) + 1`."""
        rot, theta = self.spec.rotary_dim, float(self.spec.theta)
        j = np.arange(rot // 2, dtype=np.float64)
        inv_freq = np.power(theta, -2.0 * j / rot)
        sc = getattr(self.spec, "scaling", None)
        if sc is None:
            return inv_freq, 1.0
        if hasattr(sc, "low"):
            # bands of wavelength: short ones stay, long ones turn `factor` times slower, and
            # between `original / high` and `original / low` the two are blended
            wavelength = 2.0 * np.pi / inv_freq
            blend = (sc.original / wavelength - sc.low) / (sc.high - sc.low)
            mixed = (1.0 - blend) * inv_freq / sc.factor + blend * inv_freq
            out = np.where(wavelength > sc.original / sc.low, inv_freq / sc.factor,
                           np.where(wavelength < sc.original / sc.high, inv_freq, mixed))
            return out, 1.0

        def pair_with(turns):
            return rot * np.log(sc.original / (2.0 * np.pi * turns)) / (2.0 * np.log(theta))

        low = max(np.floor(pair_with(sc.fast)), 0.0)
        high = min(np.ceil(pair_with(sc.slow)), rot - 1.0)
        ramp = np.clip((j - low) / max(high - low, 0.001), 0.0, 1.0)
        stretched = inv_freq / sc.factor * ramp + inv_freq * (1.0 - ramp)
        return stretched, sc.magnitude_slope * np.log(sc.factor) + 1.0

    def tables(self, step, head_dim):
        """(cos, sin) for a kernel that rotates on its own way (the decode attention), or None
        if this encoding is not a rotation over the whole head of positions the tables hold."""
        if self.spec.rotary_dim != head_dim or self.cos.dtype != torch.float32 \
                or step.max_position >= self.cos.shape[0]:
            return None
        return self.cos, self.sin

    def rotate_store(self, qkv, step, view, heads, kv_heads, head_dim, write_cache=True):
        if step.max_position >= self.cos.shape[0]:
            raise ValueError(f"position {step.max_position} is beyond the rotary table of "
                             f"{self.cos.shape[0]} positions")
        ops.rope_store(qkv, step.positions, step.token_seq, view.block_table, self.cos, self.sin,
                       view.keys, view.values, heads, kv_heads, head_dim, write_cache)


class RotaryInterleaved(RotaryHalf):
    """The same table of angles for pairs of neighbours: dimension 2i turns with 2i + 1. The
    kernels that take a rotation with an `interleaved` argument ask `position.interleaved`;
    the kernel behind `rotate_store` pairs halves only."""

    interleaved = True

    def tables(self, step, head_dim):
        return None

    def rotate_store(self, qkv, step, view, heads, kv_heads, head_dim, write_cache=True):
        raise NotImplementedError("rotate_store pairs (i, i + rotary_dim / 2) only")


class NoPosition(Part):
    """No position encoding: keys and values go to the cache as they are."""

    def rotate_store(self, qkv, step, view, heads, kv_heads, head_dim, write_cache=True):
        ops.rope_store(qkv, step.positions, step.token_seq, view.block_table, None, None,
                       view.keys, view.values, heads, kv_heads, head_dim, write_cache)


register_part("rotary_half", RotaryHalf)
register_part("rotary_interleaved", RotaryInterleaved)
register_part("no_position", NoPosition)
