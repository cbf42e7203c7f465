"""The kernels as Python functions over torch tensors.

Each function checks devices, types, shapes and strides, then launches on the
current CUDA stream. Nothing here computes on the host, and there is no other
implementation behind these functions: on a machine without the compiled
kernels they raise.
"""

from __future__ import annotations

import torch

from ._lib import (BF16, CACHE_BLOCK, F32, KernelError, call, dtype_code, plain_function, ptr,
                   require_cuda)
from .linear import Deferred, gated_up, linear, per_head
from . import gemm_tc
from .streams import streams_spread, streams_step, token_shift
from .recurrent import delta_rule
from .scan import causal_conv, decay_attention, norm_gate, selective_scan, step_size
from . import mixture
from .mixture import latent_prepare, rotate_heads
from .attention import (attention_decode, attention_prefill, attention_prefill_tc, decode_splits,
                        forget_descriptors,
                        fast_path_takes, kernel_errors, plan_token_blocks, plan_wide_tiles, tc_prefill_takes, upload_query_tiles,
                        upload_wide_plan)

__all__ = ["CACHE_BLOCK", "KernelError", "embed", "rms_norm", "rope_store", "attention_plain",
           "attention_decode", "attention_prefill", "attention_prefill_tc", "tc_prefill_takes", "plan_wide_tiles", "upload_wide_plan",
           "upload_query_tiles",
           "decode_splits", "plan_token_blocks", "fast_path_takes", "forget_descriptors",
           "kernel_errors", "gated_silu", "gelu_tanh", "streams_step", "streams_spread", "token_shift",
           "delta_rule", "kv_store", "layer_norm", "cached_attention", "mixture", "latent_prepare",
           "rotate_heads", "distance_attention", "rms_update", "qk_prepare", "causal_conv",
           "decay_attention", "norm_gate", "selective_scan", "step_size", "gated_up", "gemm_tc", "add_into", "scale_cap_", "linear", "per_head", "choose", "Deferred"]


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 rows of `table` for int32 `ids`; an id outside the table gives zeros."""
    require_cuda(ids, table)
    _check(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), "ids: int32 [T]")
    _check(table.dim() == 2 and table.is_contiguous(), "table: contiguous [vocab, hidden]")
    vocab, hidden = table.shape
    if out is None:
        out = torch.empty((ids.numel(), hidden), dtype=torch.float32, device=ids.device)
    _check(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (ids.numel(), hidden),
           "out: fp32 [T, hidden]")
    call("sakv_embed", ptr(ids), ptr(table), dtype_code(table.dtype), ptr(out), ids.numel(),
         hidden, vocab)
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
             rows: torch.Tensor | None = None, add: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of rows of fp32 `x`; with `rows` (int32), of those rows only. With `add`
    (fp32, x's shape or [parts, *x's shape]; bf16 weight and output) `x += add` (`+=
    add.sum(0)`, in order) happens first, in the same kernel, and x keeps the sum."""
    require_cuda(x, weight, rows, add)
    _check(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x: fp32 [T, hidden]")
    hidden = x.shape[1]
    _check(weight.shape == (hidden,) and weight.is_contiguous(), "weight: [hidden]")
    n = x.shape[0]
    if rows is not None:
        _check(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(),
               "rows: int32 [R]")
        n = rows.numel()
    if add is not None:
        _check(rows is None and add.dtype == torch.float32 and add.is_contiguous()
               and (add.shape == x.shape or (add.dim() == 3 and add.shape[1:] == x.shape))
               and weight.dtype == torch.bfloat16 and out_dtype == torch.bfloat16,
               "add: fp32 like x or [parts, *x.shape], bf16 weight and output, no rows")
    parts = add.shape[0] if add is not None and add.dim() == 3 else 1
    out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    call("sakv_rmsnorm", ptr(x), ptr(add), parts, x.numel(), ptr(rows), ptr(weight), dtype_code(weight.dtype), ptr(out),
         dtype_code(out_dtype), n, hidden, float(eps))
    return out


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
               block_table: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
               k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, heads: int,
               kv_heads: int, head_dim: int, write_cache: bool = True) -> None:
    """Rotate the queries of `qkv` in place; rotate the keys and write them and the
    values into the cache entry `k_cache`/`v_cache` ([blocks, kv_heads, 64, head_dim])."""
    require_cuda(qkv, positions, token_seq, block_table, cos, sin, k_cache, v_cache)
    tokens = qkv.shape[0]
    _check(qkv.dim() == 2 and qkv.stride(1) == 1
           and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim,
           "qkv: [T, (heads + 2 kv_heads) head_dim]")
    for t, name in ((positions, "positions"), (token_seq, "token_seq")):
        _check(t.dtype == torch.int32 and t.is_contiguous() and t.numel() == tokens,
               f"{name}: int32 [T]")
    _check(block_table.dtype == torch.int32 and block_table.dim() == 2
           and block_table.is_contiguous(), "block_table: int32 [B, max_blocks]")
    rot = 0
    if cos is not None:
        _check(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.dim() == 2
               and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape,
               "cos, sin: fp32 [positions, rot / 2]")
        rot = 2 * cos.shape[1]
    if write_cache:
        for c in (k_cache, v_cache):
            _check(c is not None and c.dtype == qkv.dtype and c.is_contiguous() and c.dim() == 4
                   and tuple(c.shape[1:]) == (kv_heads, CACHE_BLOCK, head_dim),
                   "cache entry: [blocks, kv_heads, 64, head_dim] of the activations' type")
    call("sakv_rope_store", ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0), ptr(positions),
         ptr(token_seq), ptr(block_table), block_table.shape[1], ptr(cos), ptr(sin), rot,
         ptr(k_cache), ptr(v_cache), tokens, heads, kv_heads, head_dim, int(write_cache))


def attention_plain(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                    heads: int, kv_heads: int, head_dim: int, scale: float,
                    window: int | None) -> torch.Tensor:
    """Causal grouped-query attention of every token of the step over its sequence's
    cache; queries are the first heads*head_dim columns of `qkv`."""
    require_cuda(qkv, k_cache, v_cache, positions, token_seq, block_table)
    tokens = qkv.shape[0]
    _check(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= heads * head_dim,
           "qkv: [T, >= heads * head_dim]")
    _check(head_dim <= 256, f"head_dim {head_dim}: the plain attention kernel takes up to 256")
    _check(heads % kv_heads == 0, "heads must be a multiple of kv_heads")
    for c in (k_cache, v_cache):
        _check(c.dtype == qkv.dtype and c.is_contiguous() and c.dim() == 4
               and tuple(c.shape[1:]) == (kv_heads, CACHE_BLOCK, head_dim),
               "cache entry: [blocks, kv_heads, 64, head_dim] of the activations' type")
    out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    call("sakv_attention_plain", ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0), ptr(out),
         ptr(k_cache), ptr(v_cache), ptr(positions), ptr(token_seq), ptr(block_table),
         block_table.shape[1], tokens, heads, kv_heads, head_dim, float(scale),
         int(window) if window else 0)
    return out


def gated_silu(gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up` for `gate_up[t] = [gate | up]`."""
    require_cuda(gate_up)
    _check(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0,
           "gate_up: contiguous [T, 2 * intermediate]")
    tokens, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    call("sakv_gated_silu", ptr(gate_up), ptr(out), dtype_code(gate_up.dtype), tokens, inter)
    return out


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """The tanh form of GELU, element by element (fp32 inside, x's type outside)."""
    require_cuda(x)
    _check(x.is_contiguous(), "gelu_tanh: contiguous input")
    out = torch.empty_like(x)
    call("sakv_gelu_tanh", ptr(x), ptr(out), dtype_code(x.dtype), x.numel())
    return out


def kv_store(qkv: torch.Tensor, k_off: int, v_off: int, positions: torch.Tensor,
             token_seq: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor,
             v_cache: torch.Tensor) -> None:
    """Copy a step's keys (`qkv[:, k_off:]`, kv_heads * dim wide) and values (`qkv[:, v_off:]`,
    kv_heads * vdim wide) into the cache entry: keys [blocks, kv_heads, 64, dim], values
    [blocks, kv_heads, 64, vdim]."""
    require_cuda(qkv, positions, token_seq, block_table, k_cache, v_cache)
    tokens = qkv.shape[0]
    _check(qkv.dim() == 2 and qkv.stride(1) == 1, "qkv: [T, columns] with contiguous rows")
    for c in (k_cache, v_cache):
        _check(c.dtype == qkv.dtype and c.is_contiguous() and c.dim() == 4
               and c.shape[2] == CACHE_BLOCK and c.shape[1] == k_cache.shape[1],
               "cache entry: [blocks, kv_heads, 64, width] of the activations' type")
    kv_heads, dim, vdim = k_cache.shape[1], k_cache.shape[3], v_cache.shape[3]
    _check(k_off + kv_heads * dim <= qkv.shape[1] and v_off + kv_heads * vdim <= qkv.shape[1],
           "keys or values reach beyond qkv's columns")
    _check(block_table.dtype == torch.int32 and block_table.dim() == 2
           and block_table.is_contiguous(), "block_table: int32 [B, max_blocks]")
    call("sakv_kv_store", ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0), k_off, v_off,
         ptr(positions), ptr(token_seq), ptr(block_table), block_table.shape[1], ptr(k_cache),
         ptr(v_cache), tokens, kv_heads, dim, vdim)


def distance_attention(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       positions: torch.Tensor, token_seq: torch.Tensor,
                       block_table: torch.Tensor, heads: int, scale: float, window: int | None,
                       slope: torch.Tensor | None, rate: torch.Tensor | None,
                       gate_off: int | None = None, splits: int = 1) -> torch.Tensor:
    """Causal grouped-query attention of every token of the step over its sequence's cache
    with the score `q.k * scale - slope[h] * ln(1 + rate[h] * distance)`; queries are the first
    heads * dim columns of `qkv`, and with `gate_off` each head's output is multiplied by
    `sigmoid(qkv[:, gate_off + h])`. Returns [T, heads * vdim] of qkv's type.

    `splits`: 1 (the default) scores 32 keys at a time with one warp for a token's heads of a
    key/value head, and gives a token the same result to the bit however the tokens come; more
    (up to 16) lets that many warps share a token's keys, for steps of few tokens over many
    keys; 0 is the plain form, one key at a time, which also takes widths above 256."""
    require_cuda(qkv, k_cache, v_cache, positions, token_seq, block_table, slope, rate)
    tokens = qkv.shape[0]
    kv_heads, dim, vdim = k_cache.shape[1], k_cache.shape[3], v_cache.shape[3]
    _check(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= heads * dim,
           "qkv: [T, >= heads * dim]")
    _check(heads % kv_heads == 0, "heads must be a multiple of kv_heads")
    for c in (k_cache, v_cache):
        _check(c.dtype == qkv.dtype and c.is_contiguous() and c.dim() == 4
               and c.shape[2] == CACHE_BLOCK and c.shape[1] == kv_heads,
               "cache entry: [blocks, kv_heads, 64, width] of the activations' type")
    _check((slope is None) == (rate is None), "slope and rate come together")
    for c in (slope, rate):
        _check(c is None or (c.dtype == torch.float32 and c.shape == (heads,)
                             and c.is_contiguous()), "slope, rate: fp32 [heads]")
    _check(gate_off is None or 0 <= gate_off <= qkv.shape[1] - heads, "gate_off: inside qkv")
    out = torch.empty((tokens, heads * vdim), dtype=qkv.dtype, device=qkv.device)
    call("sakv_distance_attention", ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0),
         -1 if gate_off is None else int(gate_off), ptr(out), ptr(k_cache), ptr(v_cache),
         ptr(positions), ptr(token_seq), ptr(block_table), block_table.shape[1], tokens, heads,
         kv_heads, dim, vdim, float(scale), int(window) if window else 0, ptr(slope), ptr(rate),
         int(splits))
    return out


def layer_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, out_dtype: torch.dtype,
               rows: torch.Tensor | None = None, add: torch.Tensor | None = None,
               add_weight: torch.Tensor | None = None) -> torch.Tensor | None:
    """Layer norm (weight, no bias) of rows of fp32 `x`; with `rows` (int32), of those rows
    only. With `add` (fp32, x's shape) and `add_weight`, `x += layer_norm(add) * add_weight`
    happens first, in the same kernel, and x keeps the sum; `weight` None then returns nothing
    (only the stream is completed)."""
    require_cuda(x, weight, rows, add, add_weight)
    _check(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x: fp32 [T, hidden]")
    hidden = x.shape[1]
    for w in (weight, add_weight):
        _check(w is None or (w.shape == (hidden,) and w.is_contiguous()), "weight: [hidden]")
    _check(weight is not None or add is not None, "layer_norm: nothing to do")
    _check((add is None) == (add_weight is None), "add and add_weight come together")
    if add is not None:
        _check(rows is None and add.dtype == torch.float32 and add.is_contiguous()
               and add.shape == x.shape, "add: fp32 like x, no rows")
        _check(weight is None or weight.dtype == add_weight.dtype, "the weights' types differ")
    n = x.shape[0]
    if rows is not None:
        _check(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(),
               "rows: int32 [R]")
        n = rows.numel()
    out = None if weight is None else torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    w_dtype = (weight if weight is not None else add_weight).dtype
    call("sakv_layer_norm", ptr(x), ptr(add), ptr(add_weight), ptr(rows), ptr(weight),
         dtype_code(w_dtype), ptr(out), dtype_code(out_dtype if out is not None else torch.float32),
         n, hidden, float(eps))
    return out


def rms_update(x: torch.Tensor, y: torch.Tensor | None = None,
               add_weight: torch.Tensor | None = None, add_offset: float = 0.0,
               out_dtype: torch.dtype | None = None, out_weight: torch.Tensor | None = None,
               out_offset: float = 0.0, eps: float = 0.0,
               rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """On rows of the fp32 stream `x`, in one pass: with `y` (fp32, x's shape), `x += y /
    rms(y) * (add_offset + add_weight)`; with `out_dtype`, returns the rows of x in that type,
    or with `out_weight` their RMS norm `x / rms(x) * (out_offset + out_weight)`; `rows`
    (int32; only without `y`): those rows only. rms(v) = sqrt(mean(v^2) + eps)."""
    require_cuda(x, y, add_weight, out_weight, rows)
    _check(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x: fp32 [T, hidden]")
    hidden = x.shape[1]
    for w in (add_weight, out_weight):
        _check(w is None or (w.shape == (hidden,) and w.is_contiguous()), "weight: [hidden]")
    _check(y is not None or out_dtype is not None, "rms_update: nothing to do")
    if y is not None:
        _check(rows is None and add_weight is not None and y.dtype == torch.float32
               and y.is_contiguous() and y.shape == x.shape, "y: fp32 like x, with a weight, no rows")
    _check(add_weight is None or out_weight is None or add_weight.dtype == out_weight.dtype,
           "the weights' types differ")
    n = x.shape[0]
    if rows is not None:
        _check(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(),
               "rows: int32 [R]")
        n = rows.numel()
    out = None if out_dtype is None else torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    some = add_weight if add_weight is not None else out_weight
    call("sakv_rms_update", ptr(x), ptr(y), ptr(add_weight), float(add_offset), ptr(rows),
         ptr(out_weight), float(out_offset),
         dtype_code(some.dtype) if some is not None else F32, ptr(out),
         dtype_code(out_dtype if out_dtype is not None else torch.float32), n, hidden, float(eps))
    return out


def qk_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int,
               dim: int, vdim: int, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
               eps: float, cos: torch.Tensor | None, sin: torch.Tensor | None,
               positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
               k_cache: torch.Tensor, v_cache: torch.Tensor, out_dtype: torch.dtype,
               write_cache: bool = True) -> torch.Tensor:
    """From a fused projection's fp32 output `proj` [T, columns] (queries at `q_off`, keys at
    `k_off`, values at `v_off`): queries and keys each divided by the root mean square of their
    whole projection and multiplied by `q_weight` / `k_weight` (None: no norm), the first
    `2 * cos.shape[1]` numbers of every head turned by the token's position (None: no
    rotation), keys and values stored in the cache blocks. Returns the queries [T, heads *
    dim] of `out_dtype`."""
    require_cuda(proj, q_weight, k_weight, cos, sin, positions, token_seq, block_table, k_cache,
                 v_cache)
    tokens = proj.shape[0]
    _check(proj.dtype == torch.float32 and proj.dim() == 2 and proj.stride(1) == 1,
           "proj: fp32 [T, columns] with contiguous rows")
    _check(max(q_off + heads * dim, k_off + kv_heads * dim, v_off + kv_heads * vdim)
           <= proj.shape[1], "queries, keys or values reach beyond proj's columns")
    _check((q_weight is None) == (k_weight is None), "q_weight and k_weight come together")
    if q_weight is not None:
        _check(q_weight.shape == (heads * dim,) and k_weight.shape == (kv_heads * dim,)
               and q_weight.is_contiguous() and k_weight.is_contiguous()
               and q_weight.dtype == k_weight.dtype, "norm weights: [heads * dim], [kv_heads * dim]")
    rot = 0
    if cos is not None:
        _check(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.dim() == 2
               and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape,
               "cos, sin: fp32 [positions, rot / 2]")
        rot = 2 * cos.shape[1]
    for t, name in ((positions, "positions"), (token_seq, "token_seq")):
        _check(t.dtype == torch.int32 and t.is_contiguous() and t.numel() == tokens,
               f"{name}: int32 [T]")
    _check(block_table.dtype == torch.int32 and block_table.dim() == 2
           and block_table.is_contiguous(), "block_table: int32 [B, max_blocks]")
    for c, width in ((k_cache, dim), (v_cache, vdim)):
        _check(c.dtype == out_dtype and c.is_contiguous() and c.dim() == 4
               and tuple(c.shape[1:]) == (kv_heads, CACHE_BLOCK, width),
               "cache entry: [blocks, kv_heads, 64, width] of the queries' type")
    q = torch.empty((tokens, heads * dim), dtype=out_dtype, device=proj.device)
    call("sakv_qk_prepare", ptr(proj), proj.stride(0), int(q_off), int(k_off), int(v_off),
         ptr(q_weight), ptr(k_weight), dtype_code(q_weight.dtype) if q_weight is not None else F32,
         float(eps), ptr(cos), ptr(sin), rot, ptr(positions), ptr(token_seq), ptr(block_table),
         block_table.shape[1], ptr(q), ptr(k_cache), ptr(v_cache), dtype_code(out_dtype), tokens,
         heads, kv_heads, dim, vdim, int(write_cache))
    return q


def cached_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor | None,
                     positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                     heads: int, dim: int, vdim: int, scale: float, *, maps: int = 1,
                     q2: torch.Tensor | None = None, q_split: int = 0,
                     window: int | None = None, chunk: int | None = None, lam: float = 0.0,
                     out_scale: float = 1.0, eps: float = 0.0, gate_elem_off: int | None = None,
                     splits: int = 1, key_splits: int = 1, warp_stage: bool = False,
                     heads_first: bool = False, keep_first: int = 0,
                     sink: torch.Tensor | None = None,
                     head_gate: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of every token of the step over its sequence's cache, in the general
    form of `csrc/attention_distance.cu`: scores, softmax weights and weighted sums in fp32.

    `q`: [T, heads * maps, width] with any strides between tokens and heads (a view of a
    projection's output): head h's `maps` queries are its rows h * maps .. h * maps + maps - 1,
    each `dim` columns. With `q2` ([T, heads * maps, dim - q_split], strided likewise) a query's
    columns from `q_split` on come from q2. `k_cache`: [blocks, kv_heads, 64, k_row] with map
    m's key at column m * dim; `v_cache`: [blocks, kv_heads, 64, v_row] of which the first
    `vdim` are read, or None: the values are the first `vdim` columns of the key rows. `window`
    (the last w keys) or `chunk` (keys of the query's own run of c positions) or neither;
    with a window, `keep_first` k: the keys at positions below k stay visible to every later
    query. `sink` (fp32 [heads]): the softmax's denominator of head h also holds
    `exp(sink[h])`. With one map the output is multiplied by `out_scale`, and with `head_gate`
    ([T, heads] of q's type, any row stride) head h's by `sigmoid(head_gate[t, h])`. Two
    maps are combined as `a1 - lam * a2`, divided by their root mean square over vdim (+ eps),
    times `out_scale`, times the sigmoid of the `vdim` numbers that lie `gate_elem_off + h *
    vdim` elements after the token's first query. Returns [T, heads * vdim] of q's type.
    `splits` > 1: that many warps share a token's keys (decode steps); `key_splits` > 1: that
    many blocks of such warps do (long sequences, few tokens), folding through device memory;
    `warp_stage`: each of those warps first copies a chunk's rows into shared memory, all
    copies in flight at once (where the rows' sizes allow 16-byte copies and the block's
    shared memory holds them). `heads_first` (with `splits` 1; decode steps): a block's warps
    are ONE token's groups of heads and share every chunk of its keys through shared memory, so
    the rows are read once for all the token's heads; `key_splits` blocks a token then take
    contiguous shares of the chunks."""
    require_cuda(q, k_cache, v_cache, positions, token_seq, block_table, q2, sink, head_gate)
    tokens = q.shape[0]
    _check(head_gate is None or (maps == 1 and head_gate.dtype == q.dtype and head_gate.dim() == 2
                                 and head_gate.shape == (tokens, heads)
                                 and head_gate.stride(1) == 1),
           "head_gate: [T, heads] of q's type with contiguous rows, one map")
    _check(sink is None or (sink.dtype == torch.float32 and sink.shape == (heads,)
                            and sink.is_contiguous()), "sink: fp32 [heads]")
    _check(keep_first >= 0 and not (keep_first and chunk), "keep_first goes with a window")
    _check(q.dim() == 3 and q.stride(2) == 1 and q.shape[1] == heads * maps
           and q.shape[2] >= (q_split if q2 is not None else dim),
           "q: [T, heads * maps, >= dim] with contiguous rows")
    _check(k_cache.dtype == q.dtype and k_cache.is_contiguous() and k_cache.dim() == 4
           and k_cache.shape[2] == CACHE_BLOCK, "k_cache: [blocks, kv_heads, 64, k_row] of q's type")
    kv_heads = k_cache.shape[1]
    _check(heads % kv_heads == 0, "heads must be a multiple of kv_heads")
    if v_cache is not None:
        _check(v_cache.dtype == q.dtype and v_cache.is_contiguous() and v_cache.dim() == 4
               and v_cache.shape[1] == kv_heads and v_cache.shape[2] == CACHE_BLOCK
               and v_cache.shape[3] >= vdim, "v_cache: [blocks, kv_heads, 64, >= vdim]")
    else:
        _check(k_cache.shape[3] >= vdim, "values inside the key rows: k_row >= vdim")
    if q2 is not None:
        _check(q2.dtype == q.dtype and q2.dim() == 3 and q2.stride(2) == 1
               and q2.shape[:2] == q.shape[:2] and q2.shape[2] >= dim - q_split
               and 0 <= q_split <= dim, "q2: [T, heads * maps, >= dim - q_split] of q's type")
    _check(max(q.stride(1), 0 if q2 is None else q2.stride(1)) < 2 ** 31, "head stride too large")
    _check(block_table.dtype == torch.int32 and block_table.dim() == 2
           and block_table.is_contiguous(), "block_table: int32 [B, max_blocks]")
    out = torch.empty((tokens, heads * vdim), dtype=q.dtype, device=q.device)
    scratch = tickets = None
    floats = 0
    heads_first = bool(heads_first) and splits == 1
    if key_splits > 1 and (splits > 1 or heads_first):
        groups = tokens * kv_heads * (heads * maps // kv_heads + 3)
        floats = groups * key_splits * (max(dim, vdim + 2) + 4)
        scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
        tickets = _attention_tickets.get(q.device)
        if tickets is None or tickets.numel() < groups:    # zero between calls: the last
            tickets = _attention_tickets[q.device] = torch.zeros(        # block clears its own
                max(groups, 4096), dtype=torch.int32, device=q.device)
    else:
        key_splits = 1
    call("sakv_cached_attention", ptr(q), dtype_code(q.dtype), q.stride(0), q.stride(1), ptr(q2),
         0 if q2 is None else q2.stride(0), 0 if q2 is None else q2.stride(1), q_split, -1,
         ptr(out), ptr(k_cache), k_cache.shape[3], ptr(v_cache),
         0 if v_cache is None else v_cache.shape[3], ptr(positions), ptr(token_seq),
         ptr(block_table), block_table.shape[1], tokens, heads, kv_heads, maps, dim, vdim,
         float(scale), int(window) if window else 0, int(chunk) if chunk else 0, float(lam),
         float(out_scale), float(eps), -1 if gate_elem_off is None else int(gate_elem_off),
         int(splits), int(key_splits), ptr(scratch), floats, ptr(tickets), int(warp_stage),
         int(heads_first), int(keep_first) if window else 0, ptr(sink), ptr(head_gate),
         0 if head_gate is None else head_gate.stride(0))
    return out


_attention_tickets: dict = {}


def add_into(acc: torch.Tensor, y: torch.Tensor) -> None:
    """`acc += y` with `acc` fp32; `y` of acc's shape, or [parts, *acc.shape], whose parts are
    summed first, in order (as `rms_norm(add=...)` does)."""
    require_cuda(acc, y)
    if y.dim() == acc.dim() + 1:
        total = y[0]
        if y.shape[0] > 1:
            total = y[0].clone()
            for part in y[1:]:
                add_into(total, part)
        y = total
    _check(acc.dtype == torch.float32 and acc.is_contiguous() and y.is_contiguous()
           and acc.shape == y.shape, "acc: fp32, same shape as y, both contiguous")
    call("sakv_add_into", ptr(acc), ptr(y), dtype_code(y.dtype), acc.numel())


def scale_cap_(x: torch.Tensor, scale: float = 1.0, cap: float | None = None) -> torch.Tensor:
    """In place on fp32 `x`: `x *= scale`, then with `cap` c, `x = c * tanh(x / c)`."""
    require_cuda(x)
    _check(x.dtype == torch.float32 and x.is_contiguous(), "x: contiguous fp32")
    _check(cap is None or cap > 0, "cap must be positive")
    call("sakv_scale_cap", ptr(x), x.numel(), float(scale), float(cap or 0.0))
    return x


def choose(logits: torch.Tensor, temperature: float = 0.0, seed: int = 0,
           request: torch.Tensor | None = None, step: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of fp32 `logits`: greedy at temperature 0, else a
    Gumbel-max draw keyed by (seed, request[row], step[row]). `out` (int32 [rows], contiguous):
    where to write them, instead of a new tensor."""
    require_cuda(logits, request, step, out)
    _check(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
           "logits: fp32 [rows, vocab]")
    rows, vocab = logits.shape
    if temperature > 0:
        for t, name in ((request, "request"), (step, "step")):
            _check(t is not None and t.dtype == torch.int32 and t.is_contiguous()
                   and t.numel() == rows, f"{name}: int32 [rows]")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _check(out.dtype == torch.int32 and out.shape == (rows,) and out.is_contiguous(),
               "out: int32 [rows]")
    chunks = plain_function("sakv_choose_chunks")(vocab)
    scratch = _choose_scratch.get(logits.device)
    if scratch is None or scratch[0].numel() < rows * chunks or scratch[1].numel() < rows:
        scratch = (torch.empty(max(rows * chunks, 4096), dtype=torch.int64, device=logits.device),
                   torch.zeros(max(rows, 1024), dtype=torch.int32, device=logits.device))
        _choose_scratch[logits.device] = scratch
    call("sakv_choose", ptr(logits), logits.stride(0) if rows else vocab, rows, vocab,
         float(temperature), int(seed) & 0xFFFFFFFFFFFFFFFF, ptr(request), ptr(step), ptr(out),
         ptr(scratch[0]), ptr(scratch[1]))
    return out


_choose_scratch: dict = {}
