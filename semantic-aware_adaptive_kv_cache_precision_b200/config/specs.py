"""What a model is made of, as plain data.

A configuration class (one per architecture) reads that architecture's own
config.json keys and turns them into a `ModelSpec`: a list of block
descriptions, each naming its mixer, feed-forward, norms and position encoding
with every size and constant as a field, plus the order in which the blocks
run. The parts are built from these descriptions alone; no part ever sees a
config.json or knows which architecture it belongs to.

Every spec has a `kind`: the name under which a part class is registered in
`parts.registry`. A new kind of mixer, feed-forward, norm or position encoding
is a new spec dataclass with a new `kind` and a registered part class; nothing
here needs to change for it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


class ConfigError(ValueError):
    """A config.json this library cannot run; the message names every problem."""


@dataclass(frozen=True)
class NormSpec:
    """`kind` "rms_norm": x / sqrt(mean(x^2) + eps) * w; "layer_norm": (x - mean) /
    sqrt(variance + eps) * w, no bias. `suffix` is what the norm's weight is called after
    the norm's own name (".weight" in most checkpoints, nothing in some). `offset` is added
    to the stored weight before it multiplies: 1.0 for weights stored around zero."""
    size: int
    eps: float
    kind: str = "rms_norm"
    suffix: str = ".weight"
    offset: float = 0.0


@dataclass(frozen=True)
class RampScaling:
    """Stretching of a rotation's long wavelengths for contexts beyond the one a model was
    trained on (the YaRN scheme): a pair whose wavelength makes fewer than `slow` turns in
    `original` positions has its frequency divided by `factor`, one that makes more than
    `fast` turns keeps it, and a linear ramp over the pair index lies between. Cosines and
    sines are all multiplied by `magnitude_slope * ln(factor) + 1`."""
    factor: float
    original: float
    fast: float
    slow: float
    magnitude_slope: float = 0.1


@dataclass(frozen=True)
class BandScaling:
    """Stretching of a rotation's long wavelengths by bands of wavelength (the scheme of
    Llama 3.1): a frequency f whose wavelength l = 2 pi / f is shorter than `original / high`
    stays, one longer than `original / low` becomes f / `factor`, and between the two it is
    `(1 - s) f / factor + s f` with `s = (original / l - low) / (high - low)`. Cosines and
    sines keep their size."""
    factor: float
    original: float
    low: float
    high: float


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding of the first `rotary_dim` of each head; `scaling` (a
    `RampScaling` or a `BandScaling`) stretches its long wavelengths. `kind` "rotary_half"
    pairs dimension i with i + rotary_dim / 2, "rotary_interleaved" pairs 2i with 2i + 1; the
    pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rotary_half"
    scaling: Optional[object] = None


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal self-attention over cached keys and values.

    `window` None means every earlier key is seen; a number w means the last w
    keys, the query's own included.
    """
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    qkv_bias: bool
    out_bias: bool
    scale: float
    window: Optional[int]
    position: Optional[RotarySpec]
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: `down(act(gate(x)) * up(x))`."""
    hidden: int
    intermediate: int
    activation: str
    bias: bool = False
    kind: str = "gated_mlp"
    #: the three tensors' names after the part's prefix: gate, up, down
    names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class LogDistanceAttentionSpec:
    """Grouped-query causal self-attention without a rotation: the score of query i on key
    j is `q.k * scale - slope[h] * ln(1 + rate[h] * (i - j))`, with two learned numbers a
    head, so that far keys lose weight smoothly. Values may have a width of their own
    (`value_dim`), the projections may have biases, and each head's output may be
    multiplied by a gate `sigmoid(Wg x)[h]`, one number a head, before the output
    projection. `window` as in `AttentionSpec`.

    Tensor names after the part's prefix: `q`, `k`, `v`, `o` (+ `.b` for biases), `g` for
    the gate's rows, `r1` (slopes) and `r2` (rates)."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: Optional[int]
    qkv_bias: bool = True
    out_bias: bool = True
    head_gate: bool = True
    kind: str = "log_distance_attention"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """A linear-recurrent mixer whose state, one `head_dim x head_dim` matrix a head, is
    decayed channel by channel, has the part that lies along the current unit key partly
    removed, and gets the outer product of key and value added (a delta rule with a
    removal rate a channel):

        S <- diag(w) S - (a * u)(u^T S) + k v^T,    out = S^T r

    with w = exp(-decay_scale * sigmoid(w0 + W2 tanh(W1 x))) from a low-rank pair of
    matrices of inner size `decay_rank`, a = sigmoid(Wa x + b), and u = k / sqrt(|k|^2 +
    `key_eps`). Each head's output is divided by its root mean square (`eps` inside the
    root), multiplied by a weight and by `sigmoid(Wg x)`, and projected.

    Tensor names after the part's prefix: `r`, `k`, `v`, `g`, `a`, `a.b`, `w1`, `w2`, `w0`,
    `norm`, `o`."""
    hidden: int
    heads: int
    head_dim: int
    decay_rank: int
    eps: float
    decay_scale: float = 0.6065306597126334      # exp(-1/2)
    key_eps: float = 1e-6
    kind: str = "general_delta"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are made from one cached latent a position.

    The input is projected down to `kv_rank + rot_dim` numbers: the first `kv_rank`, divided
    by their root mean square and multiplied by a weight, are the latent c; the last
    `rot_dim`, rotated by the position, are a key part that all heads share. Head h's key
    is [Wuk_h c | rotated part], its value Wuv_h c; its query [`head_dim` plain | `rot_dim`
    rotated] comes from a query latent of `q_rank` numbers (normed like c; None: straight
    from the input). The cache holds c and the rotated part only. `position.rotary_dim`
    must be `rot_dim`. `window` w: query i sees key j only if 0 <= i - j < w (None: every
    earlier key). `sink`: the softmax's denominator of head h also holds `exp(sink[h])`, a
    learned number that has no key and no value. `head_gate`: head h's output is multiplied
    by `sigmoid(Wg x)[h]`, one number a head, read from the mixer's input.

    Tensor names after the part's prefix: `dq`, `dq.norm`, `uq` (or `q` without a query
    latent), `dkv`, `dkv.norm`, `uk`, `uv`, `o`, `sink`, `g`."""
    hidden: int
    heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    q_rank: Optional[int]
    scale: float
    eps: float
    position: RotarySpec
    window: Optional[int] = None
    sink: bool = False
    head_gate: bool = False
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DifferentialAttentionSpec:
    """Grouped-query causal attention with two softmax maps a head over the same values:

        o = a1 - lam * a2,  lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff  (one number a layer)
        out = o / sqrt(mean(o^2) + eps) * (1 - diff)              (over a head's values)

    Queries are laid out head by head as [map 1 | map 2], each `head_dim` wide, keys
    likewise a key/value head. No rotation. `chunk` c: query i sees key j <= i only if both
    lie in the same run of c positions counted from the sequence's start (None: every
    earlier key). `gate`: the concatenated heads are multiplied element by element with
    `sigmoid(Wg x)` before the output projection.

    Tensor names after the part's prefix: `q`, `k`, `v`, `g`, `o`, `lq1`, `lk1`, `lq2`, `lk2`."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    chunk: Optional[int]
    diff: float
    eps: float
    gate: bool = True
    kind: str = "differential_attention"


@dataclass(frozen=True)
class ClampedExpertSpec:
    """A gated feed-forward with clamped branches: g = min(Wgate x, limit), u = clamp(Wup x,
    -limit, limit), y = g * sigmoid(alpha * g) * (u + 1), out = Wdown y."""
    intermediate: int
    limit: float
    alpha: float = 1.702


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of `experts` small feed-forwards (`e0`, `e1`, ...; all of form `expert`) of
    which each token uses the `top` with the largest router scores. `score` "sigmoid":
    each expert's score is the sigmoid of its router logit (fp32); "softmax": the softmax of
    the logits over all the router's outputs. `correction`: a learned number an output
    (`correction`) is added to the scores for the CHOICE only; the weights are the scores
    without it. `identity` n: the router has n more outputs after the experts'; an "expert"
    chosen among them has no tensors and returns its input (times the weight).
    `renormalize`: whether the chosen scores are divided by their sum. `weight_input`: the
    score multiplies the expert's input (out = sum expert(w x)) rather than its output.
    `shared`: one more expert that every token uses, multiplied by `sigmoid(Wsg x)`, one
    number a token (`shared.sg`), if `shared_gate`.

    Tensor names after the part's prefix: `router`, `correction`, `e<i>.gate`, `e<i>.up`,
    `e<i>.down`, `shared.gate`, `shared.up`, `shared.down`, `shared.sg`."""
    hidden: int
    experts: int
    top: int
    expert: ClampedExpertSpec
    shared: Optional[ClampedExpertSpec] = None
    shared_gate: bool = True
    score: str = "sigmoid"
    renormalize: bool = False
    weight_input: bool = True
    correction: bool = False
    identity: int = 0
    kind: str = "routed_experts"


@dataclass(frozen=True)
class WindowSinkAttentionSpec:
    """Grouped-query causal attention over a sliding window that also keeps a sequence's first
    tokens, with a learned logit a head in the softmax's denominator:

        query i sees key j <= i  if  i - j < window  or  j < keep_first
        weights_ij = exp(s_ij) / (sum_visible exp(s_ij') + exp(sink[h])),   s_ij = q_i . k_j * scale

    (`window` None: every earlier key; `sink` False: the plain softmax). Kept tokens keep their
    true positions. `qk_norm` "whole": queries and keys are each divided by the root mean square
    of their WHOLE projection (all heads together, `eps` inside the root) and multiplied by a
    weight of that size, before the rotation; None: no norm. `position`: a rotation of the first
    `rotary_dim` numbers of every head, or None. Values may have a width of their own; `bias`:
    q, k, v have biases. The heads' outputs are multiplied by `out_scale` before the output
    projection.

    Tensor names after the part's prefix: `q`, `k`, `v` (+ `.b`), `q.norm`, `k.norm`, `sink`, `o`."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: Optional[int]
    keep_first: int
    eps: float
    position: Optional[RotarySpec]
    sink: bool = True
    qk_norm: Optional[str] = "whole"
    bias: bool = True
    out_scale: float = 1.0
    kind: str = "window_sink_attention"


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Attention without softmax whose state, one `head_dim x value_dim` matrix a head, fades by
    a fixed factor a head:

        S <- decay[h] S + k v^T,   o = S^T q,        q, k, v = silu of their projections

    All heads' outputs together are divided by their root mean square (`eps` inside the root),
    multiplied by a weight, by `sigmoid(Wg x)` element by element (`gate`) and by `out_scale`,
    and projected.

    The variations, each a field: `activation` None leaves q, k, v as projected; `position`
    turns the first `rotary_dim` numbers of every head of q and k by the token's position;
    `key_scale` multiplies k (after the rotation); `norm` "head" divides each head's output by
    its own root mean square instead of all heads' together; `norm_weight` False: the norm has
    no weight; `gate_kind` "silu": the gate is `silu(Wg x)`.

    Tensor names after the part's prefix: `q`, `k`, `v`, `g`, `norm`, `o`."""
    hidden: int
    heads: int
    head_dim: int
    value_dim: int
    decay: tuple
    eps: float
    gate: bool = True
    out_scale: float = 1.0
    activation: Optional[str] = "silu"
    position: Optional[RotarySpec] = None
    key_scale: float = 1.0
    norm: str = "all"
    norm_weight: bool = True
    gate_kind: str = "sigmoid"
    kind: str = "decay_attention"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input; the mixer's output is the sum of
    theirs (each already multiplied by its own `out_scale`). Both must offer the branch
    interface (`input_decls`, `mix`, `w_o`): their input matrices are one product.

    Tensor names: the branches' own, after the part's prefix + `names[i]` + "."."""
    hidden: int
    left: object
    right: object
    names: tuple = ("left", "right")
    kind: str = "parallel_mixer"


@dataclass(frozen=True)
class SelectiveScanSpec:
    """The selective-scan mixer (Mamba): `[x | z] = Win h`; x passes a causal convolution a
    channel over `taps` tokens (last column: the current token; zeros before the start) and
    silu; `[dt | B | C] = Wx x` with dt `dt_rank` wide; `dt = softplus(Wdt dt + b)`, one a
    channel; `A = -exp(A_log)`; per channel c and state n

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c

    and the output is `Wo [y * silu(z)]`. State a sequence: S (fp32) and the convolution's last
    `taps - 1` inputs.

    Tensor names after the part's prefix: `in`, `conv`, `conv.b`, `x`, `dt`, `dt.b`, `A_log`,
    `D`, `o`."""
    hidden: int
    inner: int
    state: int
    dt_rank: int
    taps: int
    kind: str = "selective_scan"


@dataclass(frozen=True)
class DenseMLPSpec:
    """Dense feed-forward without a gate: `down(act(up(x)))`; tensors `up` and `down`."""
    hidden: int
    intermediate: int
    activation: str = "gelu_tanh"
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how a mixer and a feed-forward are arranged around the residual.

    `prefix` is where the block's tensors sit in the checkpoint
    ("model.layers.3."); the parts append their own names to it. `ffn` None: the layer has
    no feed-forward (and no norm before it).
    """
    prefix: str
    mixer: object
    mixer_norm: NormSpec
    ffn: object
    ffn_norm: Optional[NormSpec]
    mixer_name: str = "self_attn"
    ffn_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    ffn_norm_name: str = "post_attention_layernorm"
    kind: str = "pre_norm"


@dataclass(frozen=True)
class StreamBlockSpec:
    """A pre-norm layer over `streams` copies of the residual stream. Each sublayer reads a
    weighted sum of the streams and writes back to all of them:

        u = sum_s in[s] x_s;  y = sublayer(norm(u));  x_t <- sum_s mix[s, t] x_s + out[t] y

    (`connections` False: one stream and the plain `x += y`). With `token_shift` the
    mixer's input h is blended with the previous token's, `h + (h_prev - h) * shift`,
    element by element; the previous token's h is per-sequence state. `ffn` None: the layer
    has no feed-forward.

    Tensor names after `prefix`: the norms' (`mixer_norm_name`, `ffn_norm_name`),
    `hc1.in`, `hc1.out`, `hc1.mix` for the mixer and `hc2.*` for the feed-forward, `shift`."""
    prefix: str
    mixer: object
    mixer_norm: NormSpec
    ffn: object
    ffn_norm: Optional[NormSpec]
    streams: int = 1
    connections: bool = False
    token_shift: bool = False
    mixer_name: str = "mix"
    ffn_name: str = "mlp"
    mixer_norm_name: str = "norm1"
    ffn_norm_name: str = "norm2"
    kind: str = "stream_block"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """A layer with a norm before AND after each sublayer:

        x += norm1b(mixer(norm1(x)));   x += norm2b(ffn(norm2(x)))

    `ffn` None: the layer has no feed-forward (and no `norm2`, `norm2b`)."""
    prefix: str
    mixer: object
    ffn: object
    norm: NormSpec
    mixer_name: str = "mix"
    ffn_name: str = "mlp"
    norm_names: tuple = ("norm1", "norm1b", "norm2", "norm2b")
    kind: str = "sandwich_block"


@dataclass(frozen=True)
class OutputNormBlockSpec:
    """A layer whose sublayers read the residual stream itself and whose norms sit on the
    sublayers' OUTPUTS only:

        x += norm1(mixer(x));   x += norm2(ffn(x))

    `ffn` None: the layer has no feed-forward (and no `norm2`)."""
    prefix: str
    mixer: object
    ffn: object
    norm: NormSpec
    mixer_name: str = "mix"
    ffn_name: str = "mlp"
    norm_names: tuple = ("norm1", "norm2")
    kind: str = "output_norm_block"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block `block` with cache entry `cache`.

    A cache entry belongs to the first call that names it, which writes it;
    later calls with the same entry only read it (a layer that reads another
    layer's cache). A block may appear in several calls (a layer run twice);
    each such call needs a cache entry of its own unless it shares one on
    purpose.

    `mix_input`: before this call the stream is replaced by `W [x; x0]`, x0 being the
    embedding's output and W the model's `ModelSpec.input_mix_name` ([hidden, 2 hidden],
    the stream's columns first): how a run of layers that is repeated takes the input up
    again at the start of every pass.
    """
    block: int
    cache: int
    mix_input: bool = False


@dataclass(frozen=True)
class ModelSpec:
    """`embed_scale` multiplies the embedding's rows as they enter the residual stream;
    `logit_scale` multiplies the logits and `logit_softcap` c then bends them to
    `c * tanh(logits / c)` (None: neither); `head_bias_name` names a bias [vocab] of the
    output head. `ignore_tensors`: shell-style patterns of tensor names that a checkpoint
    of this architecture may hold without any part reading them (buffers that exporters
    write, such as a rotary table's `inv_freq`); anything else unexpected is an error."""
    architecture: str
    vocab_size: int
    hidden: int
    blocks: tuple
    run_order: tuple
    final_norm: NormSpec
    tie_head: bool
    max_positions: int
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    stop_token_ids: tuple = ()
    stored_dtype: str = "bfloat16"
    init_std: float = 0.02
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    head_bias_name: Optional[str] = None
    ignore_tensors: tuple = ()
    streams: int = 1
    input_mix_name: Optional[str] = None

    def cache_entries(self) -> int:
        return 1 + max((c.cache for c in self.run_order), default=-1)
