"""A plain, slow statement of the Nodopel decoder, one function per mechanism, token by token.

Written from the design's equations with torch tensors on the CPU, in whatever floating type the
weights are handed over in (tests use float64 or float32); nothing here is shared with the engine's
parts or kernels.  ``PlainNodopel`` keeps a request's past (the rotated keys and the values of every
execution of a layer) in a dictionary, so a prompt may be fed in any portions and must give the same
rows.

Notation: ``h`` is a sublayer's input row, ``W x`` a matrix stored ``[out, in]`` applied to a row,
``X`` the ``[streams, width]`` copies of the residual stream.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by the root of (mean of squares + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------ positions
def rotary_frequencies(rot: dict) -> list[float]:
    """One frequency per rotated pair: ``base ** (-2 i / dims)``, long wavelengths stretched by
    ``scaling.factor``, short ones kept, those between blended linearly in ``original / wavelength``."""
    dims, base = rot["dims"], rot["base"]
    scaling = rot.get("scaling")
    made = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, original = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        made.append(f)
    return made


def rotate(x: torch.Tensor, position: int, frequencies: list[float]) -> torch.Tensor:
    """The first ``2 len(frequencies)`` numbers of ``x`` rotated in pairs (i, i + half); the rest unchanged."""
    half = len(frequencies)
    out = x.clone()
    for i, f in enumerate(frequencies):
        angle = position * f
        c, s = math.cos(angle), math.sin(angle)
        u, v = x[i], x[i + half]
        out[i] = u * c - v * s
        out[i + half] = v * c + u * s
    return out


def sees(i: int, j: int, mask: dict | None) -> bool:
    """Whether the query at position i sees the key at position j: never a later one; with a mask only the
    last ``size`` positions and the first ``keep_first`` of the sequence."""
    if j > i:
        return False
    if not mask:
        return True
    size, keep = mask.get("size"), mask.get("keep_first") or 0
    return size is None or i - j < size or j < keep


# ------------------------------------------------------------------------ mixer
def differential_attention_step(w, cfg, eps, h, position, cache):
    """Two softmax maps per head over the same values, the second subtracted ``lambda`` times, the difference
    divided by its root mean square and scaled by ``1 - diff``.  ``cache``: lists 'k' (rotated keys ``[G, 2,
    dim]``) and 'v' (``[G, vdim]``), one entry a position."""
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = (w["q"] @ h + w["q.b"]).view(H, 2, d)
    k = (w["k"] @ h + w["k.b"]).view(G, 2, d)
    v = (w["v"] @ h + w["v.b"]).view(G, dv)
    rot = cfg.get("rot")
    if rot:
        frequencies = rotary_frequencies(rot)
        q = torch.stack([torch.stack([rotate(q[a, m], position, frequencies) for m in range(2)]) for a in range(H)])
        k = torch.stack([torch.stack([rotate(k[g, m], position, frequencies) for m in range(2)]) for g in range(G)])
    cache.setdefault("k", []).append(k)
    cache.setdefault("v", []).append(v)
    seen = [j for j in range(position + 1) if sees(position, j, cfg.get("mask"))]
    keys = torch.stack([cache["k"][j] for j in seen])           # [n, G, 2, d]
    values = torch.stack([cache["v"][j] for j in seen])         # [n, G, dv]
    diff = cfg["diff"]
    lam = torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff
    cap = cfg.get("softcap")
    out = []
    for head in range(H):
        g = head // (H // G)
        maps = []
        for m in range(2):
            score = (keys[:, g, m] @ q[head, m]) * cfg["scale"]
            if cap:
                score = cap * torch.tanh(score / cap)
            maps.append(torch.softmax(score, dim=0) @ values[:, g])
        o = maps[0] - lam * maps[1]
        out.append(rms(o, eps) * (1.0 - diff))
    return w["o"] @ torch.cat(out)


# ------------------------------------------------------------------------ feed-forward
def dense_feed_forward(w, h):
    return w["down"] @ (gelu_tanh(w["gate"] @ h) * (w["up"] @ h))


def expert(w, prefix, h):
    return w[prefix + "down"] @ (silu(w[prefix + "gate"] @ h) * (w[prefix + "up"] @ h))


def route(w, router, h):
    """The chosen experts (identity experts have the numbers behind the real ones) and their weights: scores
    are a softmax over all router outputs, the choice is made on score + correction, the weights are the
    chosen scores divided by their sum."""
    scores = torch.softmax(w["router"].to(torch.float64) @ h.to(torch.float64), dim=0)
    choice = scores + w["correction"].to(torch.float64)
    chosen = torch.topk(choice, router["top"]).indices.tolist()
    picked = torch.stack([scores[e] for e in chosen])
    weights = picked / (picked.sum() + 1e-20)
    return chosen, [x.to(h.dtype) for x in weights]


def experts_feed_forward(w, mlp, h):
    router = mlp["router"]
    chosen, weights = route(w, router, h)
    out = torch.zeros_like(h)
    for e, weight in zip(chosen, weights):
        out = out + weight * (expert(w, f"e{e}.", h) if e < router["experts"] else h)
    if mlp.get("shared"):
        out = out + expert(w, "shared.", h)
    return out


# ------------------------------------------------------------------------ hyper-connections
def streams_read(X, w_in):
    return (w_in[:, None] * X).sum(0)


def streams_write(X, mix, w_out, y):
    """All streams at once from the old ones: ``X'_t = sum_s mix[s, t] X_s + out[t] y``."""
    return mix.T @ X + w_out[:, None] * y[None, :]


def schedule_of(config) -> list[int]:
    """Layer numbers in the order they run: the layers of the loop ``times`` times in a row."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


class PlainNodopel:
    def __init__(self, config: dict, weights: dict[str, torch.Tensor]) -> None:
        self.config, self.w = config, weights
        self.eps = config["norm"]["eps"]
        self.schedule = schedule_of(config)
        self.past: dict = {}
        self.trail: list | None = None       # set to a list to collect the stream after every layer run

    def _part(self, prefix: str) -> dict:
        return {name[len(prefix):]: t for name, t in self.w.items() if name.startswith(prefix)}

    def step(self, request, token: int) -> torch.Tensor:
        """Feed one token of ``request``; returns its logits."""
        state = self.past.setdefault(request, {"position": 0, "caches": [dict() for _ in self.schedule]})
        position = state["position"]
        w, eps = self.w, self.eps
        streams = self.config.get("streams")
        x = w["embed"][token]
        X = x[None, :].repeat(streams, 1) if streams else None
        rows = []
        for run, index in enumerate(self.schedule):
            layer = self.config["layers"][index]
            p = f"l{index}."
            mixer = lambda h: differential_attention_step(self._part(p + "mix."), layer["mixer"], eps, h, position,
                                                          state["caches"][run])
            mlp = layer.get("mlp")
            if mlp is None:
                ff = None
            elif mlp["kind"] == "dense":
                ff = lambda h: dense_feed_forward(self._part(p + "mlp."), h)
            else:
                ff = lambda h: experts_feed_forward(self._part(p + "mlp."), mlp, h)
            for number, sublayer in ((1, mixer), (2, ff)):
                if sublayer is None:
                    continue
                norm = w[f"{p}norm{number}"]
                if streams:
                    hc = f"{p}hc{number}."
                    u = streams_read(X, w[hc + "in"])
                    X = streams_write(X, w[hc + "mix"], w[hc + "out"], sublayer(rms(u, eps) * norm))
                else:
                    x = x + sublayer(rms(x, eps) * norm)
            rows.append(X.sum(0) if streams else x)
        if self.trail is not None:
            self.trail.append(torch.stack(rows))
        state["position"] = position + 1
        final = X.sum(0) if streams else x
        return w["embed"] @ (rms(final, eps) * w["final.norm"])

    def run(self, request, tokens) -> torch.Tensor:
        return torch.stack([self.step(request, int(t)) for t in tokens])

    def forget(self, request) -> None:
        self.past.pop(request, None)
