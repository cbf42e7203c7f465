"""Small Zodirax configurations for the tests. Every size differs between them and from layer
to layer, and some take the values that make branches coincide elsewhere: one head, as many
key/value heads as heads and fewer, values wider and narrower than keys, a rotation of the
whole head and of a part, with and without stretched wavelengths (one whose bands all three
occur), windows shorter than, equal to and longer than a cache block, kept first tokens from
none to more than a block, a window so wide that nothing leaves it, decays of 1 and far below,
branch scales of 1, a convolution of one tap (no running inputs at all) and of many, a state of
one number and one wider than a warp's lanes hold four each, layers without a feed-forward,
the two kinds of layers in either order, and sizes that no vector access divides."""


def scan(inner, state, dt_rank, conv, ff):
    return {"type": "mamba1",
            "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def pair(left, right, scales, ff):
    heads, kv_heads, dim, vdim, scale, window, keep, turn = left
    r_heads, r_dim, r_vdim, decay = right
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                               "scale": scale, "mask": {"size": window, "keep_first": keep},
                               "rot": turn},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim,
                                "decay": list(decay)},
                      "left_scale": scales[0], "right_scale": scales[1]},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


MIXED = {"architecture": "Zodirax", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
         "embedding": {"scale": 2.5}, "initializer_range": 0.1,
         "layers": [pair((4, 2, 32, 24, 0.2, 37, 3, rot(10000.0, 16, (4.0, 1.0, 4.0, 64))),
                         (3, 16, 24, (0.5, 0.9, 0.995)), (0.8, 1.3), 80),
                    scan(128, 16, 6, 4, None),
                    scan(72, 5, 3, 2, 64),
                    pair((2, 2, 16, 40, 0.3, 64, 0, rot(500.0, 16)),
                         (2, 24, 8, (0.97, 0.7)), (1.0, 1.0), None)]}
ODD = {"architecture": "Zodirax", "vocab": 131, "width": 100, "norm": {"eps": 3e-6},
       "embedding": {"scale": 1.0}, "initializer_range": 0.12,
       "layers": [scan(50, 7, 5, 3, 70),
                  pair((6, 2, 20, 12, 0.25, 3, 1, rot(777.0, 6, (1.5, 0.5, 3.0, 40))),
                       (5, 12, 20, (1.0, 0.3, 0.8, 0.99, 0.6)), (1.7, 0.4), 30),
                  pair((3, 1, 24, 36, 0.18, 100, 70, rot(50.0, 24, (8.0, 1.0, 2.0, 16))),
                       (1, 36, 28, (0.9,)), (0.6, 2.0), 50),
                  scan(30, 1, 1, 1, None)]}
WIDE = {"architecture": "Zodirax", "vocab": 97, "width": 128, "norm": {"eps": 1e-6},
        "embedding": {"scale": 4.0}, "initializer_range": 0.07,
        "layers": [pair((4, 1, 128, 128, 0.088, 128, 5, rot(10000.0, 128, (32.0, 1.0, 4.0, 256))),
                        (2, 192, 64, (0.98, 0.999)), (1.0, 0.5), 192),
                   scan(256, 160, 8, 7, 128),
                   pair((1, 1, 64, 320, 0.125, 1000, 2, rot(300.0, 32)),
                        (4, 64, 128, (0.9, 0.95, 0.99, 0.999)), (1.5, 1.5), None)]}
CONFIGS = {"mixed": (MIXED, 31), "odd": (ODD, 32), "wide": (WIDE, 33)}
