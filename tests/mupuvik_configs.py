"""Small Mupuvik configurations for the tests.  They differ from one another in every size, in the order of the
layers and in every constant, and hold the cases a single model may hide: a layer without a feed-forward, a layer
that reads another layer's keys and values over a longer and over a shorter window than the owner's, values wider
and narrower than keys, one and several key/value heads, part of a head rotated, all of it, and none, one and
several chosen experts, all experts chosen, no shared expert, limits that cut and limits that never do, one and
several groups and norm parts of the scan, head sizes that are no multiple of four, and the sizes of 64 and 128 at
which the bfloat16 run takes the tensor-core attention kernels."""


def _moe(experts, top, ff, limit, shared=None):
    made = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        made["shared"] = {"ff": shared[0], "limit": shared[1]}
    return made


def _attention(heads, kv_heads, dim, vdim, scale, window, mlp, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _parallel(left, right, scales, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]},
            "mlp": mlp}


def _mamba(mixer, mlp):
    return {"type": "mamba2", "mixer": mixer, "mlp": mlp}


MV_A = {
    "architecture": "Mupuvik", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.0, "bigram": {"buckets": 53, "mul_prev": 5, "mul_cur": 3}},
    "layers": [
        _attention(4, 2, 16, 24, 0.3, 24, _moe(4, 2, 32, 0.5, (48, 1.5))),
        _attention(4, 2, 16, 24, 0.2, 40, _moe(4, 1, 24, 3.0, (16, 0.25)), kv_from=0),      # a longer window than the owner's
        _parallel({"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.35, "rot": {"base": 100.0, "dims": 8}},
                  {"heads": 2, "dim": 8, "vdim": 16, "tau": 4.0}, (0.75, 1.25), None),
        _mamba({"heads": 2, "vdim": 16, "state": 8, "groups": 1, "conv": 4, "norm_groups": 1}, _moe(3, 3, 16, 0.75)),
        _attention(4, 2, 16, 24, 0.4, 9, _moe(5, 2, 8, 1.0, (8, 1.0)), kv_from=0),          # and a shorter one
    ],
}

MV_B = {
    "architecture": "Mupuvik", "vocab": 211, "width": 96, "norm": {"eps": 1e-6},
    "embedding": {"scale": 0.25, "bigram": {"buckets": 127, "mul_prev": 1, "mul_cur": 11}},
    "layers": [
        _mamba({"heads": 6, "vdim": 8, "state": 12, "groups": 3, "conv": 2, "norm_groups": 3}, None),
        _parallel({"heads": 6, "kv_heads": 6, "dim": 20, "vdim": 12, "scale": 0.25},        # nothing rotated
                  {"heads": 3, "dim": 36, "vdim": 40, "tau": 1.0}, (1.0, 0.5), _moe(6, 1, 40, 100.0)),
        _attention(3, 3, 12, 8, 0.5, 7, _moe(2, 2, 64, 0.3, (24, 0.6))),
        _parallel({"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 40, "scale": 0.2, "rot": {"base": 7.5, "dims": 24}},
                  {"heads": 4, "dim": 12, "vdim": 8, "tau": 32.0}, (0.3, 2.0), _moe(8, 3, 16, 1.0, (32, 2.0))),
        _mamba({"heads": 4, "vdim": 12, "state": 20, "groups": 4, "conv": 3, "norm_groups": 2}, _moe(4, 1, 32, 0.5)),
    ],
}

# Keys and values of one size of 64 or 128: in bfloat16 the softmax attention runs on the tensor-core kernels.
MV_C = {
    "architecture": "Mupuvik", "vocab": 300, "width": 128, "norm": {"eps": 1e-5},
    "embedding": {"scale": 1.0, "bigram": {"buckets": 401, "mul_prev": 13, "mul_cur": 1}},
    "layers": [
        _parallel({"heads": 3, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "rot": {"base": 50000.0, "dims": 64}},
                  {"heads": 2, "dim": 40, "vdim": 72, "tau": 16.0}, (0.6, 0.9), _moe(4, 2, 64, 1.0, (96, 2.0))),
        _attention(4, 2, 64, 64, 0.125, 50, _moe(4, 1, 48, 1.0, (64, 2.0))),
        _attention(4, 2, 64, 64, 0.125, 33, None, kv_from=1),
        _mamba({"heads": 2, "vdim": 80, "state": 72, "groups": 2, "conv": 4, "norm_groups": 2}, _moe(2, 1, 96, 4.0)),
    ],
}

# Odd sizes: a width, head sizes and expert widths that are no multiple of four, a convolution of one tap, a window
# of one position (a token sees itself alone), a window longer than any sequence, large hash constants.
MV_D = {
    "architecture": "Mupuvik", "vocab": 61, "width": 50, "norm": {"eps": 1e-4},
    "embedding": {"scale": 0.5, "bigram": {"buckets": 17, "mul_prev": 1000003, "mul_cur": 998244353}},
    "layers": [
        _mamba({"heads": 3, "vdim": 7, "state": 5, "groups": 3, "conv": 1, "norm_groups": 1}, _moe(3, 2, 7, 0.5, (9, 0.5))),
        _attention(3, 3, 10, 6, 0.5, 1, _moe(2, 1, 33, 1.0)),
        _parallel({"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 6, "scale": 0.5, "rot": {"base": 3.0, "dims": 6}},
                  {"heads": 1, "dim": 6, "vdim": 9, "tau": 0.5}, (1.0, 1.0), _moe(7, 4, 5, 2.0, (3, 0.1))),
        _attention(2, 1, 14, 18, 0.3, 1000, None),
        _mamba({"heads": 2, "vdim": 9, "state": 33, "groups": 1, "conv": 5, "norm_groups": 3}, None),
    ],
}

CONFIGS = {"A": (MV_A, 16), "B": (MV_B, 8), "C": (MV_C, 32), "D": (MV_D, 4)}
LENGTHS = {
    "A": {"a": 70, "b": 45, "c": 100, "d": 37, "e": 64, "f": 1, "g": 150},
    "B": {"a": 70, "b": 33, "c": 90, "d": 2, "e": 64, "g": 130},
    "C": {"a": 70, "b": 45, "c": 130, "d": 1, "g": 200},
    "D": {"a": 41, "b": 2, "c": 23, "g": 70},
}
