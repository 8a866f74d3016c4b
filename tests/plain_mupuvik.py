"""A plain, slow statement of the Mupuvik decoder, one function per mechanism, token by token.

Everything is written from the design's equations with torch tensors on the CPU, in whatever
floating type the weights are handed over in (tests use float64 or float32); nothing here is
shared with the engine's parts or kernels.  ``PlainMupuvik`` keeps a request's state (previous
token, keys and values per layer, recurrent states, the convolution's last inputs) in a
dictionary, so a prompt may be fed in any portions and must give the same rows.

Notation: ``h`` is a mixer's input row, ``W x`` a matrix stored ``[out, in]`` applied to a row.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------ small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by the root of (mean of squares + eps), over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def bigram_row(previous: int | None, token: int, mul_prev: int, mul_cur: int, buckets: int) -> int:
    if previous is None:
        return buckets
    return (previous * mul_prev + token * mul_cur) % buckets


def embed_row(w, cfg, previous: int | None, token: int):
    bigram = cfg["embedding"]["bigram"]
    row = bigram_row(previous, token, bigram["mul_prev"], bigram["mul_cur"], bigram["buckets"])
    return w["embed"][token] * cfg["embedding"]["scale"] + w["bigram"][row]


def rotate_pairs(x: torch.Tensor, position: int, base: float, dims: int) -> torch.Tensor:
    """``x`` ``[heads, d]``: the neighbours (2i, 2i + 1) for i < dims / 2 are turned by the angle
    ``position * base ** (-2 i / dims)``; what lies behind ``dims`` stays."""
    out = x.clone()
    for i in range(dims // 2):
        angle = position * base ** (-2.0 * i / dims)
        c, s = math.cos(angle), math.sin(angle)
        u, v = x[:, 2 * i], x[:, 2 * i + 1]
        out[:, 2 * i] = u * c - v * s
        out[:, 2 * i + 1] = v * c + u * s
    return out


def attend(q, keys, values, scale: float, group: int, first_visible: int, unit_in_denominator: bool):
    """``q`` ``[H, d]``; ``keys`` ``[n, G, d]`` and ``values`` ``[n, G, dv]`` of the positions 0 .. n - 1, the last
    being the query's own.  Keys from ``first_visible`` on are seen.  With ``unit_in_denominator`` the weights
    are ``exp(s_j) / (1 + sum exp(s))``."""
    out = []
    for h in range(q.shape[0]):
        g = h // group
        scores = (keys[first_visible:, g] @ q[h]) * scale
        if unit_in_denominator:
            top = torch.clamp(scores.max(), min=0.0)
            e = torch.exp(scores - top)
            weights = e / (torch.exp(-top) + e.sum())
        else:
            weights = torch.softmax(scores, dim=0)
        out.append(weights @ values[first_visible:, g])
    return torch.stack(out)


# ------------------------------------------------------------------- the mixer 'attention'
def windowed_attention_step(w, cfg, eps, h, position, cache, lent=None):
    """Biases on q, k and v; RMS norm over all of q (and of k) at once; a window; a gate per head.
    ``lent``: another layer's cache whose keys and values are read (the layer then has none of its own)."""
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = norm_plain(w["q"] @ h + w["q.b"], w["q.norm"], eps).view(H, d)
    if lent is None:
        k = norm_plain(w["k"] @ h + w["k.b"], w["k.norm"], eps).view(G, d)
        v = (w["v"] @ h + w["v.b"]).view(G, dv)
        cache.setdefault("k", []).append(k)
        cache.setdefault("v", []).append(v)
        lent = cache
    keys, values = torch.stack(lent["k"][:position + 1]), torch.stack(lent["v"][:position + 1])
    first = max(0, position - cfg["mask"]["size"] + 1)
    o = attend(q, keys, values, cfg["scale"], H // G, first, False)
    o = o * torch.sigmoid(w["g"] @ h)[:, None]
    return w["o"] @ o.reshape(-1)


# ---------------------------------------------------------------------- the mixer 'parallel'
def rotary_sink_attention_step(w, cfg, eps, h, position, cache):
    """Left side: norm per head, neighbours rotated, causal, one added to the softmax denominator, gate per head."""
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = norm_plain((w["q"] @ h).view(H, d), w["q.norm"], eps)
    k = norm_plain((w["k"] @ h).view(G, d), w["k.norm"], eps)
    v = (w["v"] @ h).view(G, dv)
    rot = cfg.get("rot")
    if rot is not None:
        q = rotate_pairs(q, position, rot["base"], rot["dims"])
        k = rotate_pairs(k, position, rot["base"], rot["dims"])
    cache.setdefault("k", []).append(k)
    cache.setdefault("v", []).append(v)
    o = attend(q, torch.stack(cache["k"]), torch.stack(cache["v"]), cfg["scale"], H // G, 0, True)
    o = o * torch.sigmoid(w["g"] @ h)[:, None]
    return w["o"] @ o.reshape(-1)


def gated_linear_attention_step(q, k, v, alpha, state):
    """Per head: S <- diag(alpha) S + k v^T (S is ``[d, dv]``), o = S^T q."""
    out = []
    for h in range(q.shape[0]):
        state[h] = alpha[h][:, None] * state[h] + torch.outer(k[h], v[h])
        out.append(state[h].T @ q[h])
    return torch.stack(out)


def gated_linear_branch_step(w, cfg, eps, h, cache):
    H, d, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = (w["q"] @ h).view(H, d) * d ** -0.5
    k = (w["k"] @ h).view(H, d)
    v = (w["v"] @ h).view(H, dv)
    z = w["a2"] @ (w["a1"] @ h) + w["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / cfg["tau"]).view(H, d)
    if "S" not in cache:
        cache["S"] = [torch.zeros(d, dv, dtype=h.dtype) for _ in range(H)]
    o = gated_linear_attention_step(q, k, v, alpha, cache["S"])
    o = norm_plain(o, w["norm"], eps).reshape(-1) * silu(w["g"] @ h)
    return w["o"] @ o


def parallel_mixer_step(w, cfg, eps, h, position, cache):
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.")}
    a = rotary_sink_attention_step(left, cfg["left"], eps, h, position, cache.setdefault("left", {}))
    b = gated_linear_branch_step(right, cfg["right"], eps, h, cache.setdefault("right", {}))
    return cfg["left_scale"] * a + cfg["right_scale"] * b


# ------------------------------------------------------------------------ the mixer 'mamba2'
def causal_conv_step(x, weight, bias, history):
    """``weight`` ``[C, taps]``, last column for the current input; ``history`` the last taps - 1 inputs
    (oldest first, zeros before the start), updated in place."""
    taps = weight.shape[1]
    window = torch.stack(history + [x], dim=1) if taps > 1 else x[:, None]
    out = (window * weight).sum(1) + bias
    if taps > 1:
        history.pop(0)
        history.append(x)
    return out


def selective_scan_step(w, cfg, eps, h, cache):
    H, P, N, G = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"]
    inner = H * P
    row = w["in"] @ h
    z, xbc, dt = row[:inner], row[inner:2 * inner + 2 * G * N], row[2 * inner + 2 * G * N:]
    if "conv" not in cache:
        cache["conv"] = [torch.zeros_like(xbc) for _ in range(cfg["conv"] - 1)]
        cache["S"] = [torch.zeros(N, P, dtype=h.dtype) for _ in range(H)]
    xbc = silu(causal_conv_step(xbc, w["conv"], w["conv.b"], cache["conv"]))
    x = xbc[:inner].view(H, P)
    B = xbc[inner:inner + G * N].view(G, N)
    C = xbc[inner + G * N:].view(G, N)
    dt = softplus(dt + w["dt_bias"])
    y = []
    for head in range(H):
        g = head // (H // G)
        decay = torch.exp(-torch.exp(w["A_log"][head]) * dt[head])
        cache["S"][head] = decay * cache["S"][head] + dt[head] * torch.outer(B[g], x[head])
        y.append(cache["S"][head].T @ C[g] + w["D"][head] * x[head])
    y = torch.cat(y) * silu(z)
    parts = cfg["norm_groups"]
    y = rms(y.view(parts, -1), eps).reshape(-1) * w["norm"]
    return w["o"] @ y


# ------------------------------------------------------------------------------ feed-forward
def capped_expert(w, prefix, h, limit):
    g = torch.clamp(w[prefix + "gate"] @ h, max=limit)
    u = torch.clamp(w[prefix + "up"] @ h, min=-limit, max=limit)
    return w[prefix + "down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def experts_step(w, cfg, h):
    scores = torch.sigmoid(w["router"].to(h.dtype) @ h)
    top = cfg["router"]["top"]
    order = sorted(range(scores.shape[0]), key=lambda e: (-float(scores[e]), e))[:top]
    out = torch.zeros_like(h)
    for e in order:
        out = out + capped_expert(w, f"e{e}.", scores[e] * h, cfg["expert"]["limit"])
    if cfg.get("shared") is not None:
        out = out + capped_expert(w, "shared.", h, cfg["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------- model
def _under(weights, prefix):
    return {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}


class PlainMupuvik:
    """``config``: the content of config.json; ``weights``: name -> tensor (any floating type; integer tables
    as they are).  ``feed(state, tokens)`` returns the logits ``[len(tokens), vocab]`` and, with ``trail``, the
    residual after every layer."""

    def __init__(self, config: dict, weights: dict, dtype=torch.float64) -> None:
        self.cfg = config
        self.w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
        self.eps = config["norm"]["eps"]
        self.dtype = dtype
        self.layer_w = [{"mix": _under(self.w, f"l{i}.mix."), "mlp": _under(self.w, f"l{i}.mlp."),
                         "norm": _under(self.w, f"l{i}.norm")} for i in range(len(config["layers"]))]

    def new_state(self) -> dict:
        return {"previous": None, "position": 0, "layers": [{} for _ in self.cfg["layers"]]}

    def row(self, state: dict, token: int, trail: list | None = None) -> torch.Tensor:
        """The residual row of one more token (before the model's last norm)."""
        cfg, eps = self.cfg, self.eps
        x = embed_row(self.w, cfg, state["previous"], token)
        position = state["position"]
        for index, layer in enumerate(cfg["layers"]):
            w, cache, mixer = self.layer_w[index], state["layers"][index], layer["mixer"]
            h = norm_one_plus(x, w["norm"]["1"], eps)
            if layer["type"] == "attention":
                lent = state["layers"][mixer["kv_from"]] if mixer.get("kv_from") is not None else None
                y = windowed_attention_step(w["mix"], mixer, eps, h, position, cache, lent)
            elif layer["type"] == "parallel":
                y = parallel_mixer_step(w["mix"], mixer, eps, h, position, cache)
            elif layer["type"] == "mamba2":
                y = selective_scan_step(w["mix"], mixer, eps, h, cache)
            else:
                raise ValueError(layer["type"])
            x = x + norm_one_plus(y, w["norm"]["1b"], eps)
            if layer.get("mlp") is not None:
                h = norm_one_plus(x, w["norm"]["2"], eps)
                x = x + norm_one_plus(experts_step(w["mlp"], layer["mlp"], h), w["norm"]["2b"], eps)
            if trail is not None:
                trail.append(x.clone())
        state["previous"] = token
        state["position"] = position + 1
        return x

    def logits_of(self, x: torch.Tensor) -> torch.Tensor:
        return self.w["embed"] @ norm_one_plus(x, self.w["final.norm"], self.eps)

    def feed(self, state: dict, tokens, trail: list | None = None) -> torch.Tensor:
        rows = []
        for token in tokens:
            per_layer = [] if trail is not None else None
            rows.append(self.logits_of(self.row(state, int(token), per_layer)))
            if trail is not None:
                trail.append(torch.stack(per_layer))
        return torch.stack(rows)
