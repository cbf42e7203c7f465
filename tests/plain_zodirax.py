"""A plain, slow Zodirax in NumPy float64: whole sequences only, no cache, no batching, no
step function. One function for each mechanism of the design, written from its equations;
nothing here imports the package under test.

Notation: n tokens, W the model's width, H heads, G key/value heads, D a head's key size,
Dv its value size, E a mamba mixer's inner size, N its state size. Linear weights are
[out, in] and applied as `x @ w.T`.
"""

from __future__ import annotations

import math

import numpy as np

from plain_model import read_model_folder      # the tests' own safetensors reader

__all__ = ["read_model_folder", "rms_norm", "sigmoid", "silu", "softplus", "stretched_frequencies",
           "rotate_front", "causal_conv", "selective_scan", "mamba", "visible", "sink_softmax",
           "window_attention", "decayed_linear_attention", "parallel_mixer", "gated_mlp",
           "layer", "forward", "generate"]


def rms_norm(x, w, eps, plus_one=False):
    """x / sqrt(mean(x^2) + eps) * w (or * (1 + w)): eps inside the root."""
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    if w is None:
        return y
    return y * (1.0 + w) if plus_one else y * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def stretched_frequencies(rot):
    """Frequencies [dims / 2] of a rotation `rot` = {base, dims, scaling?}: f_i = base^(-2i /
    dims). With scaling {factor, low, high, original}: a wavelength l = 2 pi / f shorter than
    original / high keeps f, one longer than original / low gets f / factor, and between them
    s = (original / l - low) / (high - low) blends the two, (1 - s) f / factor + s f."""
    dims, base = rot["dims"], float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            wavelength = 2.0 * math.pi / f
            if wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wavelength >= sc["original"] / sc["high"]:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return np.array(out)


def rotate_front(x, positions, rot):
    """x: [n, heads, D]; of each head's first `dims` numbers, i is paired with i + dims/2 and
    the pair is turned by the angle position * f_i; the rest pass."""
    f = stretched_frequencies(rot)
    half = rot["dims"] // 2
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], axis=-1)


def causal_conv(x, w, b):
    """x: [n, E]; w: [E, taps], the last column multiplies the current token, the one before
    it the token before, zeros before the start; b: [E]."""
    n, taps = x.shape[0], w.shape[1]
    y = np.tile(b, (n, 1)).astype(np.float64)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            y[back:] += x[:n - back] * w[:, j]
    return y


def selective_scan(x, dt, A, B, C, D):
    """x, dt: [n, E]; A: [E, N]; B, C: [n, N]; D: [E]. S <- exp(dt A) S + dt x B^T, y = S C + D x."""
    n, E = x.shape
    S = np.zeros_like(A)
    y = np.empty((n, E))
    for t in range(n):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


def mamba(h, t, p, m):
    """`t`: tensors by name, `p`: the mixer's prefix ('l0.mix.'), `m`: its config entry."""
    E, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ t[p + "in"].T
    x, z = xz[:, :E], xz[:, E:]
    x = silu(causal_conv(x, t[p + "conv"], t[p + "conv.b"]))
    low = x @ t[p + "x"].T
    dt = softplus(low[:, :R] @ t[p + "dt"].T + t[p + "dt.b"])
    y = selective_scan(x, dt, -np.exp(t[p + "A_log"]), low[:, R:R + N], low[:, R + N:R + 2 * N],
                       t[p + "D"])
    return (y * silu(z)) @ t[p + "o"].T


def visible(n, size, keep_first):
    """[n, n] bool: query i sees key j <= i if i - j < size or j < keep_first."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def sink_softmax(s, mask, sink):
    """Softmax over the visible keys of each row whose denominator also holds exp(sink)."""
    s = np.where(mask, s, -np.inf)
    top = np.maximum(s.max(-1, keepdims=True), sink)
    e = np.exp(s - top)
    return e / (e.sum(-1, keepdims=True) + np.exp(sink - top))


def window_attention(h, t, p, m, eps):
    n = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, Dv = m.get("kv_heads", H), m.get("vdim", D)
    q = h @ t[p + "q"].T + t[p + "q.b"]
    k = h @ t[p + "k"].T + t[p + "k.b"]
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(n, G, Dv)
    q = rms_norm(q, t[p + "q.norm"], eps).reshape(n, H, D)       # over the whole projection
    k = rms_norm(k, t[p + "k.norm"], eps).reshape(n, G, D)
    pos = np.arange(n)
    if m.get("rot") is not None:
        q, k = rotate_front(q, pos, m["rot"]), rotate_front(k, pos, m["rot"])
    size, keep = (n, 0) if m.get("mask") is None else (m["mask"]["size"],
                                                         m["mask"].get("keep_first", 0))
    mask = visible(n, size, keep)
    out = np.empty((n, H, Dv))
    for head in range(H):
        g = head // (H // G)
        w = sink_softmax(q[:, head] @ k[:, g].T * m.get("scale", 1.0), mask,
                         float(t[p + "sink"][head]))
        out[:, head] = w @ v[:, g]
    return out.reshape(n, H * Dv) @ t[p + "o"].T


def decayed_linear_attention(h, t, p, m, eps):
    n = h.shape[0]
    H, D = m["heads"], m["dim"]
    Dv = m.get("vdim", D)
    q = silu(h @ t[p + "q"].T).reshape(n, H, D)
    k = silu(h @ t[p + "k"].T).reshape(n, H, D)
    v = silu(h @ t[p + "v"].T).reshape(n, H, Dv)
    o = np.empty((n, H, Dv))
    for head in range(H):
        S = np.zeros((D, Dv))
        for i in range(n):
            S = m["decay"][head] * S + np.outer(k[i, head], v[i, head])
            o[i, head] = S.T @ q[i, head]
    o = rms_norm(o.reshape(n, H * Dv), t[p + "norm"], eps) * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def parallel_mixer(h, t, p, m, eps):
    return (m.get("left_scale", 1.0) * window_attention(h, t, p + "left.", m["left"], eps)
            + m.get("right_scale", 1.0) * decayed_linear_attention(h, t, p + "right.", m["right"],
                                                                   eps))


def gated_mlp(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def layer(x, t, i, entry, eps):
    """x <- x + norm1(mixer(x)); x <- x + norm2(ff(x)): the sublayers read x itself."""
    p = f"l{i}."
    if entry["type"] == "mamba1":
        y = mamba(x, t, p + "mix.", entry["mixer"])
    elif entry["type"] == "parallel":
        y = parallel_mixer(x, t, p + "mix.", entry["mixer"], eps)
    else:
        raise ValueError(entry["type"])
    x = x + rms_norm(y, t[p + "norm1"], eps, plus_one=True)
    if entry.get("mlp") is not None:
        x = x + rms_norm(gated_mlp(x, t, p + "mlp."), t[p + "norm2"], eps, plus_one=True)
    return x


def forward(config, tensors, ids, states=None):
    """float64 logits [n, vocab]; with `states` (a list), the stream after every layer."""
    t = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][np.asarray(ids)] * (config.get("embedding") or {}).get("scale", 1.0)
    for i, entry in enumerate(config["layers"]):
        x = layer(x, t, i, entry, eps)
        if states is not None:
            states.append(x.copy())
    return rms_norm(x, t["final.norm"], eps, plus_one=True) @ t["embed"].T


def generate(config, tensors, prompt, new_tokens):
    """The `new_tokens` greedy choices after `prompt`."""
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(np.argmax(forward(config, tensors, ids)[-1])))
    return ids[len(prompt):]
