"""Small Nodopel configurations for the tests.  They differ from one another in every size, in the order of
the layers and in every constant, and hold the cases a single model may hide: one, two, four and five streams
and a model without streams, loops over the first layers, over the last, of one run and none at all, layers
without a feed-forward, values wider and narrower than keys, one and several key/value heads, layers without
a window, with windows of one and two positions, with more kept first positions than the window has and with
none, rotation over a whole map, over a part and none, frequencies on all three branches of the stretching,
scores with and without a cap, routers with more identity experts than real ones, with none, with every
expert chosen, with and without a shared expert, sizes that are no multiple of four."""


def _rot(dims, base, scaling=None):
    made = {"dims": dims, "base": base}
    if scaling is not None:
        factor, low, high, original = scaling
        made["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return made


def _layer(heads, kv_heads, dim, vdim, scale, diff, mlp, window=None, keep=None, softcap=None, rot=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        mixer["mask"] = {"size": window}
        if keep is not None:
            mixer["mask"]["keep_first"] = keep
    if softcap is not None:
        mixer["softcap"] = softcap
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, identity=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    made = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        made["shared"] = {"ff": shared}
    return made


ND_A = {
    "architecture": "Nodopel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(4, 2, 16, 24, 0.25, 0.5, _dense(80), window=20, keep=3, softcap=20.0,
               rot=_rot(8, 10000.0, (8.0, 1.0, 4.0, 64))),
        _layer(2, 2, 12, 8, 0.3, 0.8, _moe(40, 6, 2, identity=2, shared=24), window=12, keep=1, softcap=5.0,
               rot=_rot(12, 500.0)),
        _layer(4, 1, 8, 16, 0.35, 0.2, None, window=33, keep=9, rot=_rot(4, 100.0, (2.0, 1.0, 2.0, 16))),
        _layer(2, 1, 24, 24, 0.2, 0.65, _moe(24, 3, 3, identity=3), softcap=50.0, rot=_rot(24, 1.0e6)),
    ],
}

# Maps of 64 and 128 numbers, values of 64, 128 and 256; four streams, no loop; a layer without a window, one
# without rotation, one whose scores are not capped; routers without identity experts and without a shared expert.
ND_B = {
    "architecture": "Nodopel", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "streams": 4,
    "layers": [
        _layer(2, 1, 64, 128, 0.125, 0.55, _moe(32, 4, 2), window=50, keep=5, softcap=25.0,
               rot=_rot(32, 40000.0, (6.0, 1.0, 4.0, 128))),
        _layer(2, 2, 64, 64, 0.125, 0.3, _dense(96), rot=_rot(64, 10000.0)),
        _layer(1, 1, 128, 256, 0.09, 0.7, _moe(16, 8, 4, identity=0, shared=64), window=70, keep=0, softcap=15.0),
        _layer(4, 2, 128, 128, 0.09, 0.4, _dense(64), window=17, keep=2, rot=_rot(64, 2000.0, (16.0, 2.0, 8.0, 256))),
    ],
}

# Odd sizes: a width, maps, values and feed-forward widths that are no multiple of four; one stream; windows of
# one and of two positions; more kept positions than the window has; more identity experts than real ones; a loop
# over the last layers.
ND_C = {
    "architecture": "Nodopel", "vocab": 61, "width": 50, "norm": {"eps": 1e-4}, "streams": 1,
    "loop": {"start": 2, "stop": 4, "times": 3},
    "layers": [
        _layer(3, 3, 10, 6, 0.5, 0.9, _moe(33, 2, 3, identity=5), window=2, keep=6, softcap=8.0, rot=_rot(6, 30.0)),
        _layer(3, 1, 6, 10, 0.45, 0.1, _moe(9, 5, 5, shared=7), window=1, keep=4, rot=_rot(2, 7.0)),
        _layer(6, 2, 6, 14, 0.3, 0.55, _dense(77), window=9, keep=1, softcap=2.0),
        _layer(1, 1, 22, 18, 0.3, 0.35, None, window=25, rot=_rot(10, 900.0, (3.0, 0.5, 1.5, 20))),
    ],
}

# No streams at all (a plain residual), a loop over the first layer alone, layers without a feed-forward in the
# middle and at the end.
ND_D = {
    "architecture": "Nodopel", "vocab": 40, "width": 96, "norm": {"eps": 1e-5},
    "loop": {"start": 0, "stop": 1, "times": 3},
    "layers": [
        _layer(6, 3, 16, 16, 0.25, 0.45, _moe(24, 12, 3, identity=4, shared=40), window=40, keep=8, softcap=12.0,
               rot=_rot(16, 3000.0, (5.0, 1.0, 3.0, 32))),
        _layer(3, 1, 16, 32, 0.25, 0.3, None, window=30, keep=2, rot=_rot(16, 700.0)),
        _layer(2, 1, 32, 48, 0.2, 0.75, _dense(120), window=64, keep=16, rot=_rot(8, 250.0)),
        _layer(2, 2, 8, 12, 0.4, 0.15, None, window=21),
    ],
}

# Wider: products over a width that the kernels for few rows take whole, five streams, sixteen experts and eight
# identity experts, a loop of one run, pages of 32.
ND_E = {
    "architecture": "Nodopel", "vocab": 500, "width": 384, "norm": {"eps": 1e-5}, "streams": 5,
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        _layer(6, 3, 64, 64, 0.125, 0.35, _dense(448), window=100, keep=7, softcap=35.0,
               rot=_rot(48, 20000.0, (8.0, 1.0, 4.0, 512))),
        _layer(12, 1, 32, 48, 0.18, 0.25, _moe(96, 16, 4, identity=8, shared=160), window=130, keep=33, softcap=40.0,
               rot=_rot(32, 5000.0)),
        _layer(3, 3, 48, 80, 0.15, 0.5, _moe(160, 16, 6, identity=2), rot=_rot(16, 800.0, (2.0, 1.0, 4.0, 64))),
    ],
}

CONFIGS = {"A": (ND_A, 16), "B": (ND_B, 16), "C": (ND_C, 4), "D": (ND_D, 8), "E": (ND_E, 32)}
LENGTHS = {
    "A": {"a": 70, "b": 45, "c": 100, "d": 37, "e": 64, "f": 1, "g": 150},
    "B": {"a": 70, "b": 33, "c": 130, "d": 2, "e": 64, "g": 200},
    "C": {"a": 41, "b": 2, "c": 23, "g": 70},
    "D": {"a": 70, "b": 1, "c": 140, "g": 230},
    "E": {"a": 300, "b": 64, "c": 129, "g": 260},
}
