"""A mixture of gated feed-forwards routed on the device (`csrc/moe.cu`), and the small ops
around attention over a cached latent (`csrc/latent.cu`)."""

from __future__ import annotations

import torch

from ._lib import KernelError, call, dtype_code, plain_function, ptr, require_cuda


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


class Routing:
    """What `route` leaves on the device for one step's tokens: for every (token, choice)
    the expert, its weight and the row it has among the experts' sorted input rows; where
    each expert's rows begin; and the tiles of the grouped products."""

    __slots__ = ("tokens", "top", "experts", "chosen", "weights", "rank", "slot_of", "offsets",
                 "tile_expert", "tile_row", "n_tiles", "max_tiles")


_counts: dict = {}

#: up to this many tokens one block chooses for all of them and plans, in one launch
ROUTE_IN_ONE_BLOCK = 64


def tile_rows() -> int:
    return plain_function("sakv_moe_tile_rows")()


def router_logits(h: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """fp32 [T, outputs] = h weight^T with fp32 `weight` [outputs, width] and fp32 sums, h
    [T, width] in either type: the router's product, 32-bit in both modes."""
    require_cuda(h, weight)
    _check(h.dim() == 2 and h.is_contiguous() and weight.dtype == torch.float32
           and weight.is_contiguous() and weight.dim() == 2 and weight.shape[1] == h.shape[1],
           "h: contiguous [T, width]; weight: fp32 [outputs, width]")
    out = torch.empty((h.shape[0], weight.shape[0]), dtype=torch.float32, device=h.device)
    call("sakv_moe_logits", ptr(h), dtype_code(h.dtype), ptr(weight), ptr(out), h.shape[0],
         weight.shape[0], h.shape[1])
    return out


def route(logits: torch.Tensor, experts: int, top: int, identity: int = 0,
          softmax: bool = False, bias: torch.Tensor | None = None) -> Routing:
    """logits: fp32 [T, >= experts + identity]; the `top` largest scores among the first
    `experts + identity` columns a row. The score is the sigmoid of the logit, or with
    `softmax` the softmax over those columns; `bias` (fp32 [experts + identity]) is added for
    the choice only. A choice among the last `identity` columns is an identity expert: it gets
    no row in the grouped products, and `combine` adds the token's input times its weight."""
    require_cuda(logits, bias)
    outputs = experts + identity
    _check(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
           and logits.shape[1] >= outputs, "logits: fp32 [T, >= experts + identity]")
    _check(bias is None or (bias.dtype == torch.float32 and bias.shape == (outputs,)
                            and bias.is_contiguous()), "bias: fp32 [experts + identity]")
    tokens, dev = logits.shape[0], logits.device
    key = (dev, experts)
    counts = _counts.get(key)
    if counts is None:        # zero between steps: the plan kernel clears what it has read
        counts = _counts[key] = torch.zeros(experts, dtype=torch.int32, device=dev)
    r = Routing()
    r.tokens, r.top, r.experts = tokens, top, experts
    ints = torch.empty((3, tokens, top), dtype=torch.int32, device=dev)
    r.chosen, r.rank, r.slot_of = ints[0], ints[1], ints[2]
    r.weights = torch.empty((tokens, top), dtype=torch.float32, device=dev)
    r.max_tiles = -(-tokens * top // tile_rows()) + min(experts, tokens * top)
    plan = torch.empty(experts + 2 + 2 * r.max_tiles, dtype=torch.int32, device=dev)
    r.offsets, r.n_tiles = plan[:experts + 1], plan[experts + 1:experts + 2]
    r.tile_expert = plan[experts + 2:experts + 2 + r.max_tiles]
    r.tile_row = plan[experts + 2 + r.max_tiles:]
    if 0 < tokens <= ROUTE_IN_ONE_BLOCK:
        call("sakv_moe_route_plan", ptr(logits), logits.stride(0), outputs, top, ptr(r.chosen),
             ptr(r.weights), ptr(r.rank), tokens, experts, int(bool(softmax)), ptr(bias),
             ptr(r.offsets), ptr(r.tile_expert), ptr(r.tile_row), ptr(r.n_tiles), r.max_tiles)
        return r
    call("sakv_moe_route", ptr(logits), logits.stride(0), outputs, top, ptr(r.chosen),
         ptr(r.weights), ptr(counts), ptr(r.rank), tokens, experts, int(bool(softmax)), ptr(bias))
    call("sakv_moe_plan", ptr(counts), ptr(r.offsets), ptr(r.tile_expert), ptr(r.tile_row),
         ptr(r.n_tiles), experts, r.max_tiles)
    return r


def gather_rows(h: torch.Tensor, r: Routing, weight_input: bool) -> torch.Tensor:
    """The experts' input rows [T * top, width], sorted by expert: h's rows, times the
    choice's weight if `weight_input`."""
    require_cuda(h)
    _check(h.dim() == 2 and h.is_contiguous() and h.shape[0] == r.tokens, "h: contiguous [T, width]")
    rows = torch.empty((r.tokens * r.top, h.shape[1]), dtype=h.dtype, device=h.device)
    call("sakv_moe_gather", ptr(h), dtype_code(h.dtype), ptr(r.chosen), ptr(r.weights),
         ptr(r.rank), ptr(r.offsets), ptr(rows), ptr(r.slot_of), r.tokens, r.top, h.shape[1],
         int(weight_input))
    return rows


def grouped_product(rows: torch.Tensor, r: Routing, w0: torch.Tensor, w1: torch.Tensor | None,
                    limit: float = 0.0, alpha: float = 0.0) -> torch.Tensor:
    """rows [R, k] sorted by expert times every expert's own weights. `w0`, `w1`: [experts, n,
    k]. With `w1`: the clamped gated activation of the two products, [R, n] of rows' type;
    without: the product, fp32 [R, n]."""
    require_cuda(rows, w0, w1)
    _check(rows.dim() == 2 and rows.is_contiguous() and w0.dim() == 3 and w0.is_contiguous()
           and w0.shape[0] == r.experts and w0.shape[2] == rows.shape[1]
           and w0.dtype == rows.dtype, "rows [R, k], weights [experts, n, k] of one type")
    _check(w1 is None or (w1.shape == w0.shape and w1.is_contiguous() and w1.dtype == w0.dtype
                          and w1.stride() == w0.stride()), "w1: like w0")
    n, k = w0.shape[1], w0.shape[2]
    out = torch.empty((rows.shape[0], n), dtype=rows.dtype if w1 is not None else torch.float32,
                      device=rows.device)
    call("sakv_moe_product", ptr(rows), dtype_code(rows.dtype), ptr(w0), ptr(w1), w0.stride(0),
         ptr(r.tile_expert), ptr(r.tile_row), ptr(r.offsets), ptr(r.n_tiles), r.max_tiles,
         ptr(out), n, k, int(w1 is not None), float(limit), float(alpha))
    return out


def clamped_act(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """`g * sigmoid(alpha g) * (u + 1)` with g = min(gate, limit), u = clamp(up, +-limit) for
    `gate_up[t] = [gate | up]`."""
    require_cuda(gate_up)
    _check(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0,
           "gate_up: contiguous [T, 2 ff]")
    tokens, ff = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((tokens, ff), dtype=gate_up.dtype, device=gate_up.device)
    call("sakv_clamped_act", ptr(gate_up), ptr(out), dtype_code(gate_up.dtype), tokens, ff,
         float(limit), float(alpha))
    return out


def combine(products: torch.Tensor, r: Routing, weight_output: bool,
            shared: torch.Tensor | None = None, gate: torch.Tensor | None = None,
            h: torch.Tensor | None = None, into: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 [T, width]: every token's rows of `products` (fp32 [T * top, width]) summed in the
    order of its choices (times their weights if `weight_output`), plus `shared` (fp32 [T,
    width]) times `sigmoid(gate)` (`gate`: fp32 [T], may be strided; None: times 1). `h` ([T,
    width], the experts' input): what a chosen identity expert adds, times its weight. `into`
    (fp32 [T, width], the residual stream): the sum is added to it and it is returned."""
    require_cuda(products, shared, gate, h, into)
    width = products.shape[1]
    if h is None:
        h = products            # (read only for identity experts, which then do not occur)
    _check(h.is_contiguous() and h.shape[1] == width and h.shape[0] >= r.tokens,
           "h: contiguous [T, width]")
    _check(products.dtype == torch.float32 and products.is_contiguous()
           and products.shape[0] == r.tokens * r.top, "products: fp32 [T * top, width]")
    _check(shared is None or (shared.dtype == torch.float32 and shared.is_contiguous()
                              and shared.shape == (r.tokens, width)), "shared: fp32 [T, width]")
    _check(gate is None or (gate.dtype == torch.float32 and gate.dim() == 1
                            and gate.shape[0] == r.tokens), "gate: fp32 [T]")
    _check(into is None or (into.dtype == torch.float32 and into.is_contiguous()
                            and into.shape == (r.tokens, width)), "into: fp32 [T, width]")
    out = into if into is not None else torch.empty((r.tokens, width), dtype=torch.float32,
                                                    device=products.device)
    call("sakv_moe_combine", ptr(products), ptr(r.slot_of), ptr(r.weights), int(weight_output),
         ptr(shared), ptr(gate), 0 if gate is None else gate.stride(0), ptr(out), r.tokens, r.top,
         width, ptr(h), dtype_code(h.dtype), int(into is not None))
    return out


def latent_prepare(down: torch.Tensor, q_rank: int, rank: int, rot: int,
                   q_weight: torch.Tensor | None, kv_weight: torch.Tensor, eps: float, step, view,
                   cos: torch.Tensor, sin: torch.Tensor, act_dtype: torch.dtype,
                   write_cache: bool = True, interleaved: bool = False) -> torch.Tensor | None:
    """From the fused down projection `down` (fp32 [T, q_rank + rank + rot]): the normed query
    latent [T, q_rank] of `act_dtype` (None if q_rank is 0), and into the cache entry `view`
    (keys [blocks, 1, 64, rank + rot]) the normed latent and the rotated shared key part
    (pairs (i, i + rot/2); `interleaved`: (2i, 2i + 1))."""
    require_cuda(down, q_weight, kv_weight, cos, sin, view.keys)
    tokens = down.shape[0]
    _check(down.dtype == torch.float32 and down.dim() == 2 and down.stride(1) == 1
           and down.shape[1] >= q_rank + rank + rot, "down: fp32 [T, q_rank + rank + rot]")
    _check(cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
           and cos.shape == sin.shape and cos.shape[1] == rot // 2, "cos, sin: fp32 [positions, rot/2]")
    keys = view.keys
    _check(keys.dtype == act_dtype and keys.is_contiguous()
           and tuple(keys.shape[1:]) == (1, 64, rank + rot),
           "cache entry: [blocks, 1, 64, rank + rot] of the activations' type")
    _check(kv_weight.dtype == act_dtype and (q_rank == 0 or q_weight.dtype == act_dtype),
           "norm weights of the activations' type")
    q_latent = torch.empty((tokens, q_rank), dtype=act_dtype, device=down.device) if q_rank else None
    call("sakv_latent_prepare", ptr(down), down.stride(0), q_rank, rank, rot, ptr(q_weight),
         ptr(kv_weight), dtype_code(act_dtype), float(eps), ptr(step.positions),
         ptr(step.token_seq), ptr(view.block_table), view.block_table.shape[1], ptr(cos), ptr(sin),
         ptr(q_latent), ptr(keys), dtype_code(act_dtype), int(write_cache), int(interleaved),
         tokens)
    return q_latent


def rotate_heads(x: torch.Tensor, head_stride: int, offset: int, heads: int, rot: int,
                 positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 interleaved: bool = False) -> None:
    """In place: in every head of every row of `x`, the `rot` columns from `offset` on are
    rotated by the row's position (pairs (i, i + rot/2); `interleaved`: (2i, 2i + 1))."""
    require_cuda(x, positions, cos, sin)
    _check(x.dim() == 2 and x.stride(1) == 1, "x: [T, columns] with contiguous rows")
    _check(cos.shape[1] == rot // 2 and cos.dtype == torch.float32 and cos.is_contiguous()
           and sin.is_contiguous(), "cos, sin: fp32 [positions, rot/2]")
    call("sakv_rotate_heads", ptr(x), dtype_code(x.dtype), x.stride(0), head_stride, offset, heads,
         rot, ptr(positions), ptr(cos), ptr(sin), int(interleaved), x.shape[0])
