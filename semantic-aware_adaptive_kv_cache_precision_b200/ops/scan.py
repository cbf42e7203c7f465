"""The recurrences without feedback from the state into its own update, over a step's tokens
(`csrc/recurrent_scan.cu`): the selective scan with its convolution and step sizes, and
attention without softmax over a fading state with its norm and gate."""

from __future__ import annotations

import torch

from ._lib import KernelError, call, dtype_code, ptr, require_cuda


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def causal_conv(xz: torch.Tensor, channels: int, weight: torch.Tensor,
                bias: torch.Tensor | None, state: torch.Tensor, step, out_dtype: torch.dtype,
                keep_state: bool = True) -> torch.Tensor:
    """silu of the causal convolution a channel over the first `channels` columns of fp32 `xz`
    [T, columns]: `weight` [channels, taps], whose last column multiplies the token itself.
    `state`: fp32 [slots, taps - 1, channels], each sequence's last inputs, read and (with
    `keep_state`) replaced. Returns [T, channels] of `out_dtype`."""
    require_cuda(xz, weight, bias, state)
    tokens, taps = xz.shape[0], weight.shape[1]
    _check(xz.dtype == torch.float32 and xz.dim() == 2 and xz.stride(1) == 1
           and xz.shape[1] >= channels, "xz: fp32 [T, >= channels] with contiguous rows")
    _check(weight.shape == (channels, taps) and weight.is_contiguous(), "weight: [channels, taps]")
    _check(bias is None or (bias.shape == (channels,) and bias.is_contiguous()
                            and bias.dtype == weight.dtype), "bias: [channels] of the weight's type")
    _check(state.dtype == torch.float32 and state.is_contiguous()
           and tuple(state.shape[1:]) == (taps - 1, channels),
           "state: fp32 [slots, taps - 1, channels]")
    out = torch.empty((tokens, channels), dtype=out_dtype, device=xz.device)
    if getattr(step, "is_decode", False) and tokens == step.sequences:
        # every sequence brings one token: output and running inputs in one launch
        call("sakv_conv_step", ptr(xz), xz.stride(0), ptr(weight), ptr(bias),
             dtype_code(weight.dtype), ptr(state), ptr(step.slots), ptr(out),
             dtype_code(out_dtype), tokens, channels, taps, int(keep_state))
        return out
    call("sakv_causal_conv", ptr(xz), xz.stride(0), ptr(weight), ptr(bias),
         dtype_code(weight.dtype), ptr(state), ptr(step.cu_seqlens), ptr(step.token_seq),
         ptr(step.slots), ptr(out), dtype_code(out_dtype), tokens, channels, taps)
    if keep_state and taps > 1:
        call("sakv_conv_state", ptr(xz), xz.stride(0), ptr(state), ptr(step.cu_seqlens),
             ptr(step.slots), step.sequences, channels, taps)
    return out


def step_size(low: torch.Tensor, rank: int, weight: torch.Tensor,
              bias: torch.Tensor | None) -> torch.Tensor:
    """fp32 [T, channels] = softplus(low[:, :rank] weight^T + bias), all in fp32."""
    require_cuda(low, weight, bias)
    channels = weight.shape[0]
    _check(low.dtype == torch.float32 and low.dim() == 2 and low.stride(1) == 1
           and low.shape[1] >= rank, "low: fp32 [T, >= rank] with contiguous rows")
    _check(weight.shape == (channels, rank) and weight.is_contiguous(), "weight: [channels, rank]")
    _check(bias is None or (bias.shape == (channels,) and bias.is_contiguous()
                            and bias.dtype == weight.dtype), "bias: [channels] of the weight's type")
    dt = torch.empty((low.shape[0], channels), dtype=torch.float32, device=low.device)
    call("sakv_step_size", ptr(low), low.stride(0), int(rank), ptr(weight), ptr(bias),
         dtype_code(weight.dtype), ptr(dt), low.shape[0], channels)
    return dt


def selective_scan(x: torch.Tensor, dt: torch.Tensor | None, low: torch.Tensor, b_off: int,
                   c_off: int, n_state: int, z: torch.Tensor, a_log: torch.Tensor,
                   d_skip: torch.Tensor, state: torch.Tensor, step, keep_state: bool = True,
                   run: int = 0, dt_weight: torch.Tensor | None = None,
                   dt_bias: torch.Tensor | None = None) -> torch.Tensor:
    """`S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c`
    over each sequence's tokens, A = -exp(a_log); returns `y * silu(z)` [T, channels] of x's
    type. `x`: [T, channels]; `dt`: fp32 [T, channels]; B and C: `n_state` columns of fp32
    `low` from `b_off` and `c_off`; `z`: fp32 [T, channels] (a view with any row stride);
    `state`: fp32 [slots, channels, n_state], read and (with `keep_state`) left.

    `run` 0: one walk over each sequence's tokens, so the sums do not depend on how a sequence
    was cut into steps. `run` r > 0: a sequence's tokens are walked in runs of r side by side
    (three launches: the runs from zero, the states carried from run to run, the runs again
    with their outputs); `step.max_new` bounds a sequence's tokens.

    `dt` None (a step of few tokens, one walk): the kernel makes the step sizes itself,
    `softplus(low[:, :rank] dt_weight^T + dt_bias)` with `dt_weight` [channels, rank] of
    a_log's type, adding the products in the order `step_size` adds them."""
    require_cuda(x, dt, low, z, a_log, d_skip, state, dt_weight, dt_bias)
    tokens, channels = x.shape
    rank = 0
    if dt is None:
        _check(not run and dt_weight is not None and dt_weight.dim() == 2
               and dt_weight.shape[0] == channels and dt_weight.is_contiguous()
               and dt_weight.dtype == a_log.dtype and dt_weight.shape[1] <= low.shape[1]
               and (dt_bias is None or (dt_bias.shape == (channels,) and dt_bias.is_contiguous()
                                        and dt_bias.dtype == a_log.dtype)),
               "without dt: dt_weight [channels, rank] (and dt_bias [channels]) of a_log's type, "
               "one walk")
        rank = dt_weight.shape[1]
    _check(x.is_contiguous() and (dt is None or (dt.dtype == torch.float32 and dt.is_contiguous()
                                                 and dt.shape == x.shape)),
           "x: [T, channels]; dt: fp32 of the same shape")
    _check(low.dtype == torch.float32 and low.dim() == 2 and low.stride(1) == 1
           and max(b_off, c_off) + n_state <= low.shape[1] and low.shape[0] == tokens,
           "low: fp32 [T, columns] holding B and C")
    _check(z.dtype == torch.float32 and z.shape == x.shape and z.stride(1) == 1,
           "z: fp32 [T, channels] with contiguous rows")
    _check(a_log.shape == (channels, n_state) and a_log.is_contiguous()
           and d_skip.shape == (channels,) and d_skip.is_contiguous()
           and d_skip.dtype == a_log.dtype, "a_log: [channels, n_state]; d_skip: [channels]")
    _check(state.dtype == torch.float32 and state.is_contiguous()
           and tuple(state.shape[1:]) == (channels, n_state), "state: fp32 [slots, channels, n_state]")
    out = torch.empty_like(x)
    runs, scratch, sums = _runs(run, step, channels * n_state, channels, x.device)
    call("sakv_selective_scan", ptr(x), dtype_code(x.dtype), ptr(dt), ptr(low), low.stride(0),
         int(b_off), int(c_off), ptr(z), z.stride(0), ptr(a_log), ptr(d_skip),
         dtype_code(a_log.dtype), ptr(state), ptr(step.cu_seqlens), ptr(step.slots), ptr(out),
         tokens, step.sequences, channels, n_state, int(keep_state), int(run) if runs else 0,
         runs, ptr(scratch), ptr(sums), ptr(dt_weight), ptr(dt_bias), int(rank))
    return out


def _runs(run: int, step, state_size: int, sum_size: int, device):
    """(runs a sequence at most, scratch for every run's state, scratch for its sums) of a
    step walked in runs of `run` tokens; (0, None, None) where one walk does."""
    if not run:
        return 0, None, None
    runs = -(-int(step.max_new) // int(run))
    if runs <= 1 or step.sequences * runs > 65535:
        return 0, None, None
    scratch = torch.empty((step.sequences * runs, state_size), dtype=torch.float32, device=device)
    sums = torch.empty((step.sequences * runs, sum_size), dtype=torch.float32,
                       device=device) if sum_size else None
    return runs, scratch, sums


def decay_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, dim: int,
                    vdim: int, decay_less_one: torch.Tensor, state: torch.Tensor, step,
                    keep_state: bool = True, run: int = 0, activation: bool = True,
                    cos: torch.Tensor | None = None, sin: torch.Tensor | None = None,
                    key_scale: float = 1.0) -> torch.Tensor:
    """`S <- decay[h] S + k v^T; o = S^T q` a head over each sequence's tokens, with q, k, v =
    silu of the columns of fp32 `proj` from `q_off`, `k_off` (heads * dim each) and `v_off`
    (heads * vdim), or those columns as they are (`activation` False). With `cos`, `sin` (fp32
    [positions, rot / 2]) the first rot numbers of every head of q and k are turned by the
    token's position (pairs (i, i + rot / 2)); `key_scale` multiplies k after that.
    `decay_less_one`: fp32 [heads] holding `decay - 1` (the kernel adds `(decay - 1) S + k
    v^T` to S). `state`: fp32 [slots, heads, vdim, dim] (the state's transpose), read and (with
    `keep_state`) left. `run`: as in `selective_scan`. Returns fp32 [T, heads * vdim]."""
    require_cuda(proj, decay_less_one, state, cos, sin)
    rot = 0
    if cos is not None:
        _check(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
               and cos.dim() == 2 and cos.is_contiguous() and sin.is_contiguous()
               and cos.shape == sin.shape and 2 * cos.shape[1] <= dim,
               "cos, sin: fp32 [positions, rot / 2] with rot <= dim")
        rot = 2 * cos.shape[1]
    tokens = proj.shape[0]
    _check(proj.dtype == torch.float32 and proj.dim() == 2 and proj.stride(1) == 1
           and max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim) <= proj.shape[1],
           "proj: fp32 [T, columns] holding q, k and v")
    _check(decay_less_one.dtype == torch.float32 and decay_less_one.shape == (heads,)
           and decay_less_one.is_contiguous(), "decay_less_one: fp32 [heads]")
    _check(state.dtype == torch.float32 and state.is_contiguous()
           and tuple(state.shape[1:]) == (heads, vdim, dim), "state: fp32 [slots, heads, vdim, dim]")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=proj.device)
    runs, scratch, _ = _runs(run, step, heads * vdim * dim, 0, proj.device)
    call("sakv_decay_attention", ptr(proj), proj.stride(0), int(q_off), int(k_off), int(v_off),
         ptr(decay_less_one), ptr(state), ptr(step.cu_seqlens), ptr(step.slots), ptr(out), tokens,
         step.sequences, heads, dim, vdim, int(keep_state), int(run) if runs else 0, runs,
         ptr(scratch), int(bool(activation)), rot, ptr(step.positions) if rot else None, ptr(cos),
         ptr(sin), float(key_scale))
    return out


def norm_gate(y: torch.Tensor, weight: torch.Tensor | None, gate: torch.Tensor | None, eps: float,
              scale: float, out_dtype: torch.dtype, group: int | None = None,
              gate_silu: bool = False) -> torch.Tensor:
    """`y / sqrt(mean(y^2) + eps) * weight * sigmoid(gate) * scale` over whole rows of fp32 `y`
    [T, width], or with `group` over each run of that many numbers of a row (a head's
    outputs); `weight` None: no weight; `gate`: fp32 [T, width] (a view with any row stride)
    or None, used as `gate * sigmoid(gate)` with `gate_silu`."""
    require_cuda(y, weight, gate)
    tokens, width = y.shape
    group = width if group is None else int(group)
    _check(y.dtype == torch.float32 and y.is_contiguous(), "y: contiguous fp32 [T, width]")
    _check(weight is None or (weight.shape == (width,) and weight.is_contiguous()),
           "weight: [width]")
    _check(group > 0 and width % group == 0, "group: a divisor of the width")
    _check(gate is None or (gate.dtype == torch.float32 and gate.shape == y.shape
                            and gate.stride(1) == 1), "gate: fp32 [T, width] with contiguous rows")
    out = torch.empty((tokens, width), dtype=out_dtype, device=y.device)
    call("sakv_norm_gate", ptr(y), ptr(weight),
         dtype_code(weight.dtype if weight is not None else torch.float32), ptr(gate),
         0 if gate is None else gate.stride(0), ptr(out), dtype_code(out_dtype), tokens, width,
         group, int(bool(gate_silu)), float(eps), float(scale))
    return out
