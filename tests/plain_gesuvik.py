"""A plain, slow Gesuvik in NumPy float64: whole sequences only, no cache, no batching, no step
function. One function for each mechanism of the design, written from its equations; nothing
here imports the package under test.

Notation: n tokens, W the model's width, H heads, G key/value heads, D a head's key size, Dv
its value size, C the latent's size, R the rotated size. Linear weights are [out, in] and
applied as `x @ w.T`.
"""

from __future__ import annotations

import math

import numpy as np

from plain_model import read_model_folder      # the tests' own safetensors reader

__all__ = ["read_model_folder", "rms_norm", "sigmoid", "silu", "frequencies", "turn_halves",
           "turn_neighbours", "banded", "sink_softmax", "retention", "latent_attention",
           "attention", "clamped_expert", "route", "experts", "layer", "forward", "generate",
           "owner"]

ALPHA = 1.702          # the experts' activation: g * sigmoid(ALPHA g)
MAGNITUDE = 0.1        # stretched rotations grow cos and sin by MAGNITUDE ln(factor) + 1


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) (* w): eps inside the root."""
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def frequencies(rot):
    """(f [dims / 2], magnitude) of a rotation {base, dims, scaling?}: f_i = base^(-2i / dims).
    With scaling {factor, original, fast, slow}: p(t) = dims ln(original / (2 pi t)) / (2 ln
    base); lo = max(floor(p(fast)), 0), hi = min(ceil(p(slow)), dims - 1); r_i = clip((i - lo)
    / max(hi - lo, 0.001), 0, 1); f_i <- f_i / factor * r_i + f_i (1 - r_i); the magnitude is
    MAGNITUDE ln(factor) + 1, otherwise 1."""
    dims, base = rot["dims"], float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def p(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(p(sc["fast"])), 0)
    hi = min(math.ceil(p(sc["slow"])), dims - 1)
    r = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * r + f * (1.0 - r), MAGNITUDE * math.log(sc["factor"]) + 1.0


def _cos_sin(positions, rot):
    f, size = frequencies(rot)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    return np.cos(a) * size, np.sin(a) * size


def turn_halves(x, positions, rot):
    """x: [n, heads, D]; of each head's first `dims` numbers, i is paired with i + dims/2 and
    the pair (u, v) becomes (u cos - v sin, v cos + u sin); the rest pass."""
    cos, sin = _cos_sin(positions, rot)
    half = rot["dims"] // 2
    cos, sin = cos[:, None, :], sin[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], axis=-1)


def turn_neighbours(x, positions, rot):
    """As `turn_halves`, with 2i paired with 2i + 1."""
    cos, sin = _cos_sin(positions, rot)
    dims = rot["dims"]
    cos, sin = cos[:, None, :], sin[:, None, :]
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def banded(n, size):
    """[n, n] bool: query i sees key j if 0 <= i - j < size (size None: every j <= i)."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    seen = j <= i
    return seen if size is None else seen & (i - j < size)


def sink_softmax(scores, seen, sink):
    """scores: [n, n]; softmax over the seen keys of each row whose denominator also holds
    exp(sink) (None: the plain softmax)."""
    s = np.where(seen, scores, -np.inf)
    top = s.max(-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink)
    e = np.where(seen, np.exp(s - top), 0.0)
    total = e.sum(-1, keepdims=True)
    if sink is not None:
        total = total + np.exp(sink - top)
    return e / total


def retention(h, t, p, m, eps):
    """Linear attention with a fixed decay a head: S <- decay S + k v^T, o = S^T q; q, k turned
    (halves), k times D^(-1/2) afterwards; each head's o over its root mean square; times
    silu(g); Wo."""
    n = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = (h @ t[p + "q"].T).reshape(n, H, D)
    k = (h @ t[p + "k"].T).reshape(n, H, D)
    v = (h @ t[p + "v"].T).reshape(n, H, Dv)
    if m.get("rot"):
        q, k = turn_halves(q, pos, m["rot"]), turn_halves(k, pos, m["rot"])
    k = k * D ** -0.5
    o = np.zeros((n, H, Dv))
    for a in range(H):
        S = np.zeros((D, Dv))
        for i in range(n):
            S = m["decay"][a] * S + np.outer(k[i, a], v[i, a])
            o[i, a] = S.T @ q[i, a]
    o = rms_norm(o, None, eps).reshape(n, H * Dv)
    return (o * silu(h @ t[p + "g"].T)) @ t[p + "o"].T


def latent_attention(h, t, p, m, eps):
    """Attention whose keys and values come from one latent a position: the first C rows of
    Wdkv h, normed, are c; the last R, turned (neighbours), are a key part all heads share.
    Head a: key [Wuk_a c | shared], value Wuv_a c, query [D plain | R turned]; window, sink,
    a gate sigmoid(Wg h)_a a head; Wo."""
    n = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n)
    rot = dict(m["rot"], dims=R)
    q = (h @ t[p + "q"].T).reshape(n, H, D + R)
    q_plain, q_turn = q[..., :D], turn_neighbours(q[..., D:], pos, rot)
    down = h @ t[p + "dkv"].T
    c = rms_norm(down[:, :C], t[p + "dkv.norm"], eps)
    shared = turn_neighbours(down[:, None, C:], pos, rot)[:, 0]
    keys = (c @ t[p + "uk"].T).reshape(n, H, D)
    values = (c @ t[p + "uv"].T).reshape(n, H, Dv)
    seen = banded(n, (m.get("mask") or {}).get("size"))
    gate = sigmoid(h @ t[p + "g"].T) if p + "g" in t else None
    out = np.zeros((n, H, Dv))
    for a in range(H):
        s = (q_plain[:, a] @ keys[:, a].T + q_turn[:, a] @ shared.T) * m["scale"]
        w = sink_softmax(s, seen, t[p + "sink"][a] if p + "sink" in t else None)
        out[:, a] = w @ values[:, a]
        if gate is not None:
            out[:, a] *= gate[:, a:a + 1]
    return out.reshape(n, H * Dv) @ t[p + "o"].T


def attention(h, t, p, m, eps):
    """Grouped-query attention: q and k normed over their whole projection, turned (halves,
    the first `dims` of every head), window, sink; Wo."""
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = rms_norm(h @ t[p + "q"].T, t[p + "q.norm"], eps).reshape(n, H, D)
    k = rms_norm(h @ t[p + "k"].T, t[p + "k.norm"], eps).reshape(n, G, D)
    v = (h @ t[p + "v"].T).reshape(n, G, Dv)
    if m.get("rot"):
        q, k = turn_halves(q, pos, m["rot"]), turn_halves(k, pos, m["rot"])
    seen = banded(n, (m.get("mask") or {}).get("size"))
    out = np.zeros((n, H, Dv))
    for a in range(H):
        g = a // (H // G)
        s = q[:, a] @ k[:, g].T * m["scale"]
        out[:, a] = sink_softmax(s, seen, t[p + "sink"][a] if p + "sink" in t else None) @ v[:, g]
    return out.reshape(n, H * Dv) @ t[p + "o"].T


def clamped_expert(h, t, p, limit):
    g = np.minimum(h @ t[p + "gate"].T, limit)
    u = np.clip(h @ t[p + "up"].T, -limit, limit)
    return (g * sigmoid(ALPHA * g) * (u + 1.0)) @ t[p + "down"].T


def route(h, t, p, top):
    """(chosen [n, top], weights [n, top]): softmax over all the router's outputs; the `top`
    largest of score + correction are chosen (ties: the lowest index), weighted by the score
    itself."""
    z = h @ t[p + "router"].T
    e = np.exp(z - z.max(-1, keepdims=True))
    s = e / e.sum(-1, keepdims=True)
    choice = s + t[p + "correction"] if p + "correction" in t else s
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def experts(h, t, p, mlp):
    """Routed experts, of which the last `identity` have no tensors and return their input,
    plus a shared expert for every token."""
    r = mlp["router"]
    chosen, weights = route(h, t, p, r["top"])
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        for e, w in zip(chosen[i], weights[i]):
            if e >= r["experts"]:
                out[i] += w * h[i]
            else:
                out[i] += w * clamped_expert(h[i:i + 1], t, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_expert(h, t, p + "shared.", mlp["shared"]["limit"])
    return out


MIXERS = {"retention": retention, "latent_attention": latent_attention, "attention": attention}


def owner(config, i):
    """The layer whose tensors layer i uses."""
    return config["layers"][i].get("weights_of", i)


def layer(x, t, config, i):
    entry = config["layers"][i]
    p, eps = f"l{owner(config, i)}.", config["norm"]["eps"]
    x = x + MIXERS[entry["type"]](rms_norm(x, t[p + "norm1"], eps), t, p + "mix.", entry["mixer"], eps)
    if entry.get("mlp"):
        x = x + experts(rms_norm(x, t[p + "norm2"], eps), t, p + "mlp.", entry["mlp"])
    return x


def forward(config, tensors, ids, hidden_states=None):
    """float64 logits [n, vocab] of one whole sequence; with `hidden_states` (a list), the
    stream after every layer is appended to it."""
    t = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    x = t["embed"][np.asarray(ids)]
    for i in range(len(config["layers"])):
        x = layer(x, t, config, i)
        if hidden_states is not None:
            hidden_states.append(x.copy())
    z = rms_norm(x, t["final.norm"], config["norm"]["eps"]) @ t["head"].T
    z = z * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z


def generate(config, tensors, ids, new_tokens):
    """The `new_tokens` tokens that greedy decoding adds to `ids`."""
    ids = list(ids)
    for _ in range(new_tokens):
        ids.append(int(np.argmax(forward(config, tensors, ids)[-1])))
    return ids[len(ids) - new_tokens:]
