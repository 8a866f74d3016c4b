"""Mupuvik: a decoder whose layers mix tokens by windowed attention, by two mixers side by side (rotary softmax
attention with a unit sink beside gated linear attention) or by a selective scan, and whose feed-forwards are
mixtures of capped experts, as a description made of parts.

What the design fixes, and so what is written here rather than read from config.json:

* the embedding is a token row times ``embedding.scale`` plus a row of a hashed table of (previous token, token) pairs;
* every layer is ``h += post(mixer(pre(h)))`` and, where it has one, ``h += post(ff(pre(h)))``, with all four norms
  (and the model's last one) RMSNorm whose stored vector lies around zero (weight ``1 + w``);
* ``attention``: biased projections, RMSNorm over all of q and over all of k with plain weights, no rotation, a
  window, an ordinary softmax, a sigmoid gate per head from the mixer's input; a layer may read the keys and values
  an earlier layer cached;
* ``parallel``: left, per-head RMSNorm of queries and keys with one plain weight vector, neighbours ``(2i, 2i + 1)``
  rotated, causal, one added to the softmax denominator, a sigmoid gate per head; right, linear attention whose
  state decays per key channel by ``sigmoid(z) ** (1 / tau)``, a norm per head, a silu gate; the two are added with
  ``left_scale`` and ``right_scale``;
* ``mamba2``: the selective scan with silu, softplus step sizes and the gate ahead of its grouped norm;
* an expert is ``down(g sigmoid(1.702 g) (u + 1))`` with ``g = min(gate h, limit)`` and ``u = clamp(up h, -limit,
  limit)``; router scores are sigmoids, the weights are the chosen scores as they are and multiply the expert's
  input; a shared expert of the same form runs for every token;
* the logits are the embedding table (unscaled) times the normalised stream.

Tensor names: ``embed``, ``bigram``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down``, ``final.norm``; matrices are stored ``[out, in]``.
"""

from __future__ import annotations

import math

import torch

from ..config.bemuzen_config import Mamba2MixerConfig
from ..config.mupuvik_config import MupuvikConfig, ParallelMixerConfig, WindowedAttentionConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

SWISH_SLOPE = 1.702         # of an expert's gate
UP_OFFSET = 1.0             # added to an expert's capped up projection


def _norm(config: MupuvikConfig, name: str) -> PartSpec:
    # The tensor is the norm's own name (no ".weight" behind it) and is stored around zero.
    return PartSpec("rms_norm", {"eps": config.norm_eps, "offset": 1.0, "weight_name": ""}, name=name)


def _longest(windows) -> int | None:
    """The window a cache must keep for layers that read it over these windows."""
    windows = list(windows)
    return None if any(w is None for w in windows) else max(windows)


def _mixer(config: MupuvikConfig, index: int) -> tuple[PartSpec, PartSpec]:
    """The layer's mixer and the position encoding it is handed."""
    mixer = config.layers[index].mixer
    none = PartSpec("none")
    if isinstance(mixer, Mamba2MixerConfig):
        return PartSpec("selective_scan", {
            "num_heads": mixer.heads, "value_dim": mixer.vdim, "state_dim": mixer.state, "groups": mixer.groups,
            "conv_taps": mixer.conv, "norm_groups": mixer.norm_groups, "norm_eps": config.norm_eps,
        }, name="mix"), none
    if isinstance(mixer, WindowedAttentionConfig):
        readers = [other.mixer.window for other in config.layers
                   if isinstance(other.mixer, WindowedAttentionConfig) and other.mixer.kv_from == index]
        return PartSpec("gated_softmax_attention", {
            "num_heads": mixer.heads, "num_kv_heads": mixer.kv_heads, "head_dim": mixer.dim, "value_dim": mixer.vdim,
            "scale": mixer.scale, "window": mixer.window, "cache_window": _longest([mixer.window, *readers]),
            "bias": True, "qk_norm": "whole", "qk_norm_eps": config.norm_eps, "unit_sink": False,
            "output_gate": True, "own_kv": mixer.kv_from is None,
        }, name="mix"), none
    left, right = mixer.left, mixer.right
    softmax = PartSpec("gated_softmax_attention", {
        "num_heads": left.heads, "num_kv_heads": left.kv_heads, "head_dim": left.dim, "value_dim": left.vdim,
        "scale": left.scale, "window": None, "bias": False, "qk_norm": "head", "qk_norm_eps": config.norm_eps,
        "unit_sink": True, "output_gate": True,
    }, name="left")
    linear = PartSpec("gated_linear_attention", {
        "num_heads": right.heads, "head_dim": right.dim, "value_dim": right.vdim, "tau": right.tau,
        "norm_eps": config.norm_eps,
    }, name="right")
    position = none if left.rot_base is None else PartSpec(
        "rotary", {"theta": left.rot_base, "rotary_dim": left.rot_dims, "interleaved": True})
    return PartSpec("paired_mixers", {"branches": (softmax, linear), "combine": "weighted_sum",
                                      "scales": (mixer.left_scale, mixer.right_scale)}, name="mix"), position


def _feed_forward(mlp) -> PartSpec:
    params = {
        "num_experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "correction": False,
        "scoring": "sigmoid", "renormalise": False, "weight_on_input": True,
        "activation": ("capped", mlp.limit, SWISH_SLOPE, UP_OFFSET),
    }
    if mlp.shared_ff is not None:
        params.update({"shared_intermediate_size": mlp.shared_ff,
                       "shared_activation": ("capped", mlp.shared_limit, SWISH_SLOPE, UP_OFFSET)})
    return PartSpec("routed_experts", params, name="mlp")


def build_spec(config: MupuvikConfig) -> ModelSpec:
    layers, schedule = [], []
    for index, layer in enumerate(config.layers):
        norms = {"mixer": _norm(config, "norm1"), "post_mixer": _norm(config, "norm1b")}
        feed_forward = None
        if layer.mlp is not None:
            norms.update({"feed_forward": _norm(config, "norm2"), "post_feed_forward": _norm(config, "norm2b")})
            feed_forward = _feed_forward(layer.mlp)
        mixer, position = _mixer(config, index)
        layers.append(LayerSpec(name=f"l{index}", block=PartSpec("sandwich_norm"), mixer=mixer,
                                feed_forward=feed_forward, position=position, norms=norms))
        # one execution per layer, so a layer's number is also its place in the schedule
        schedule.append(ScheduleEntry(layer=index, cache_from=getattr(layer.mixer, "kv_from", None)))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("bigram_embedding", {
            "buckets": config.bigram_buckets, "mul_prev": config.bigram_mul_prev, "mul_cur": config.bigram_mul_cur,
            "scale": config.embedding_scale, "weight_names": ("embed", "bigram")}, name=""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(config, "final.norm"),
        output_head=PartSpec("linear_head", {"tied": True}, name="head"),
    )


def random_weights(config: MupuvikConfig, seed: int, *, std: float | None = None, norm_std: float = 0.1,
                   decay_rank: int = 16, dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu"
                   ) -> dict[str, torch.Tensor]:
    """Seeded random tensors under the checkpoint's names: matrices ``N(0, std)`` (``std`` defaults to ``fan_in **
    -0.5``, which keeps activations of order one through any width), vectors stored around zero ``N(0, norm_std)``,
    plain norm weights ``1 + N(0, norm_std)``, biases ``N(0, 0.1)``, the decay's bias spread around 2 (decays near
    one), ``A_log`` and ``dt_bias`` spread so that the heads' decays differ.  ``decay_rank``: the rank of the two small
    matrices of the gated linear branch, which no configuration key names."""
    generator = torch.Generator(device=device).manual_seed(seed)

    def normal(shape, mean: float, spread: float) -> torch.Tensor:
        return (mean + torch.empty(shape, dtype=torch.float32, device=device).normal_(
            0.0, 1.0, generator=generator) * spread).to(dtype)

    def matrix(rows: int, cols: int) -> torch.Tensor:
        return normal((rows, cols), 0.0, std if std is not None else 1.0 / math.sqrt(cols))

    hidden = config.hidden_size
    weights = {"embed": normal((config.vocab_size, hidden), 0.0, 1.0),
               "bigram": normal((config.bigram_buckets + 1, hidden), 0.0, 0.5)}
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.mlp is not None else ()):
            weights[p + name] = normal((hidden,), 0.0, norm_std)
        mixer = layer.mixer
        if isinstance(mixer, Mamba2MixerConfig):
            inner = mixer.heads * mixer.vdim
            channels = inner + 2 * mixer.groups * mixer.state
            weights[p + "mix.in"] = matrix(inner + channels + mixer.heads, hidden)
            weights[p + "mix.conv"] = normal((channels, mixer.conv), 0.0, 0.5)
            weights[p + "mix.conv.b"] = normal((channels,), 0.0, 0.1)
            weights[p + "mix.dt_bias"] = normal((mixer.heads,), -1.0, 1.0)
            weights[p + "mix.A_log"] = normal((mixer.heads,), 0.0, 1.0)
            weights[p + "mix.D"] = normal((mixer.heads,), 1.0, 0.3)
            weights[p + "mix.norm"] = normal((inner,), 1.0, norm_std)
            weights[p + "mix.o"] = matrix(hidden, inner)
        elif isinstance(mixer, WindowedAttentionConfig):
            rows = {"q": mixer.heads * mixer.dim}
            if mixer.kv_from is None:
                rows.update({"k": mixer.kv_heads * mixer.dim, "v": mixer.kv_heads * mixer.vdim})
            for name, count in rows.items():
                weights[p + f"mix.{name}"] = matrix(count, hidden)
                weights[p + f"mix.{name}.b"] = normal((count,), 0.0, 0.1)
                if name != "v":
                    weights[p + f"mix.{name}.norm"] = normal((count,), 1.0, norm_std)
            weights[p + "mix.g"] = matrix(mixer.heads, hidden)
            weights[p + "mix.o"] = matrix(hidden, mixer.heads * mixer.vdim)
        else:
            assert isinstance(mixer, ParallelMixerConfig)
            left, right = mixer.left, mixer.right
            weights[p + "mix.left.q"] = matrix(left.heads * left.dim, hidden)
            weights[p + "mix.left.k"] = matrix(left.kv_heads * left.dim, hidden)
            weights[p + "mix.left.v"] = matrix(left.kv_heads * left.vdim, hidden)
            weights[p + "mix.left.q.norm"] = normal((left.dim,), 1.0, norm_std)
            weights[p + "mix.left.k.norm"] = normal((left.dim,), 1.0, norm_std)
            weights[p + "mix.left.g"] = matrix(left.heads, hidden)
            weights[p + "mix.left.o"] = matrix(hidden, left.heads * left.vdim)
            keys = right.heads * right.dim
            weights[p + "mix.right.q"] = matrix(keys, hidden)
            weights[p + "mix.right.k"] = matrix(keys, hidden)
            weights[p + "mix.right.v"] = matrix(right.heads * right.vdim, hidden)
            weights[p + "mix.right.g"] = matrix(right.heads * right.vdim, hidden)
            weights[p + "mix.right.o"] = matrix(hidden, right.heads * right.vdim)
            weights[p + "mix.right.norm"] = normal((right.vdim,), 1.0, norm_std)
            weights[p + "mix.right.a1"] = matrix(decay_rank, hidden)
            weights[p + "mix.right.a2"] = matrix(keys, decay_rank)
            weights[p + "mix.right.a2.b"] = normal((keys,), 2.0, 1.0)
        mlp = layer.mlp
        if mlp is not None:
            weights[p + "mlp.router"] = matrix(mlp.experts, hidden)
            for expert in range(mlp.experts):
                weights[p + f"mlp.e{expert}.gate"] = matrix(mlp.ff, hidden)
                weights[p + f"mlp.e{expert}.up"] = matrix(mlp.ff, hidden)
                weights[p + f"mlp.e{expert}.down"] = matrix(hidden, mlp.ff)
            if mlp.shared_ff is not None:
                weights[p + "mlp.shared.gate"] = matrix(mlp.shared_ff, hidden)
                weights[p + "mlp.shared.up"] = matrix(mlp.shared_ff, hidden)
                weights[p + "mlp.shared.down"] = matrix(hidden, mlp.shared_ff)
    weights["final.norm"] = normal((hidden,), 0.0, norm_std)
    return weights


register_architecture("Mupuvik", MupuvikConfig, build_spec, random_weights)
