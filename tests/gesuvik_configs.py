"""Small Gesuvik configurations for the tests. Every size differs between them and from layer
to layer, and some take the values that make branches coincide elsewhere: one head, as many
key/value heads as heads and fewer, values wider and narrower than keys, a rotation of the whole
head, of a part and none, with and without stretched wavelengths, windows shorter than, equal
to and longer than a cache block and none at all, decays of 1 and far below, one expert a token
and several, as many choices as the router has outputs, identity experts from none to several,
with and without a shared expert, layers without a feed-forward, layers that run with an
earlier layer's weights (of every kind of mixer), the kinds of layers in any order, and sizes
that no vector access divides."""


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def moe(experts, identity, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top},
           "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def retention(heads, dim, vdim, decay, turn, mlp):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if turn is not None:
        mixer["rot"] = turn
    return {"type": "retention", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, window, base, mlp):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": scale, "rot": rot(base, rot_dim)}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, window, turn, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if turn is not None:
        mixer["rot"] = turn
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def again(layer, source):
    """A layer that runs with layer `source`'s weights: the same entry, marked."""
    return dict(layer, weights_of=source)


_M0 = latent(4, 16, 8, 24, 40, 0.2, 37, 10000.0, moe(6, 2, 2, 48, 1.0, (32, 3.0)))
MIXED = {"architecture": "Gesuvik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
         "logit_scale": 1.5, "logit_softcap": 20.0, "initializer_range": 0.12,
         "layers": [_M0,
                    retention(3, 16, 24, (0.5, 0.9, 0.995), rot(1000.0, 8), None),
                    attention(4, 2, 32, 24, 0.2, 64, rot(10000.0, 16, (4.0, 64, 8.0, 2.0)),
                              moe(5, 0, 5, 40, 0.7)),
                    again(_M0, 0),
                    retention(2, 24, 8, (1.0, 0.7), rot(50.0, 24), moe(3, 1, 1, 64, 2.5))]}
_O0 = attention(6, 2, 20, 12, 0.25, 3, rot(777.0, 6, (1.5, 40, 4.0, 0.5)),
                moe(7, 3, 3, 22, 0.8, (30, 2.0)))
_O1 = retention(5, 12, 20, (1.0, 0.3, 0.8, 0.99, 0.6), None, moe(3, 0, 2, 50, 1.5))
ODD = {"architecture": "Gesuvik", "vocab": 131, "width": 100, "norm": {"eps": 3e-6},
       "logit_softcap": 9.0, "initializer_range": 0.1,
       "layers": [_O0, _O1, again(_O0, 0),
                  latent(5, 12, 6, 20, 36, 0.25, 100, 777.0, None),
                  attention(3, 3, 24, 36, 0.2, None, None, None),
                  again(_O1, 1)]}
WIDE = {"architecture": "Gesuvik", "vocab": 97, "width": 128, "norm": {"eps": 1e-6},
        "logit_scale": 3.0, "initializer_range": 0.07,
        "layers": [retention(2, 192, 64, (0.98, 0.999), rot(10000.0, 64),
                             moe(4, 1, 2, 128, 7.0, (64, 7.0))),
                   latent(2, 128, 64, 128, 512, 0.07, 128, 10000.0, None),
                   attention(4, 1, 128, 320, 0.088, 1000,
                             rot(10000.0, 128, (32.0, 256, 32.0, 1.0)), moe(9, 0, 4, 32, 1.0)),
                   retention(4, 64, 128, (0.9, 0.95, 0.99, 0.999), rot(300.0, 32), None),
                   latent(1, 8, 32, 8, 16, 0.3, None, 100.0, moe(2, 2, 1, 96, 1.2, (16, 1.0)))]}
CONFIGS = {"mixed": (MIXED, 41), "odd": (ODD, 42), "wide": (WIDE, 43)}


def rows_agree(got, want, dtype, what=""):
    """`got` [rows, columns] from the engine against float64 `want`, row by row. The design
    has places where rounding is amplified (a retention head's output is divided by its own
    root mean square, so among a sequence's first tokens, where it is one or a few products
    q.k times a value, a q.k that nearly cancels leaves its sign to the last bits), so a few
    rows may stand out; a fault of a mechanism moves most rows, and by far more.

    float32: a row's largest difference over its largest size is within 2e-5 for 97 rows of a
    hundred and within 1e-3 for all. bfloat16: the root mean square of a row's differences
    over the row's spread has a median within 0.05, nine rows of ten within 0.15 (the kernels
    alone are held to a hundredth). Fewer than eight rows: each within 1e-4, or 0.15."""
    import numpy as np
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: values that are not finite"
    diff = got - want
    if len(diff) < 8:
        err = np.abs(diff).max(-1) / np.abs(want).max(-1) if dtype == "float32" \
            else np.sqrt((diff * diff).mean(-1)) / want.std(-1)
        assert err.max() <= (1e-4 if dtype == "float32" else 0.15), \
            f"{what}: row {int(err.argmax())} differs by {err.max():.2e}"
        return
    if dtype == "float32":
        err = np.abs(diff).max(-1) / np.abs(want).max(-1)
        assert np.quantile(err, 0.97) <= 2e-5 and err.max() <= 1e-3, \
            f"{what}: row {int(err.argmax())} differs by {err.max():.2e} of its size, " \
            f"97 of 100 rows within {np.quantile(err, 0.97):.2e}"
        return
    err = np.sqrt((diff * diff).mean(-1)) / want.std(-1)
    assert np.median(err) <= 0.05 and np.quantile(err, 0.9) <= 0.15, \
        f"{what}: the median row differs by {np.median(err):.3f} of its spread, nine of ten " \
        f"within {np.quantile(err, 0.9):.3f}, the worst (row {int(err.argmax())}) {err.max():.3f}"
