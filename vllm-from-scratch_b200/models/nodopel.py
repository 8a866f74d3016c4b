"""Nodopel: a decoder whose residual is kept as several streams that every sublayer reads as a weighted sum
and updates by a small mixing matrix (hyper-connections), whose attention has two softmax maps to a head
(the second subtracted from the first), whose feed-forwards are dense or routed with identity experts and a
shared expert, and some of whose layers run several times in a row, as a description made of parts.

What the design fixes, and so what is written here rather than read from config.json:

* a layer is pre-norm, ``x += mixer(norm1(x))`` then ``x += ff(norm2(x))``, with RMSNorms of a plain weight; with
  streams, sublayer q reads ``u = sum_s in_q[s] X_s`` and updates ``X_t <- sum_s mix_q[s, t] X_s + out_q[t]
  sublayer(norm(u))``; every stream starts as the embedding's row and the last norm reads their plain sum;
* the mixer is differential attention with two maps (``parts/attention.py``): biases on the projections of
  queries, keys and values, rotate-half rotation of the first ``rot.dims`` numbers of every map with the
  stretching of long wavelengths, capped scores, a window that keeps the first positions, ``o = a1 - lambda a2``
  with ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, a norm of the head's output without a weight and the
  factor ``1 - diff``;
* the dense feed-forward is ``down(gelu_tanh(gate h) * (up h))``; an expert (the shared one too) is
  ``down(silu(gate h) * (up h))``; the router's scores are a softmax over all its outputs, the choice is made on
  score + correction, the weights are the chosen scores divided by their sum; the last ``identity`` outputs of
  the router stand for experts that return their input;
* the layers ``loop.start .. loop.stop - 1`` run ``loop.times`` times in a row with the same weights, every run
  with a cache of its own;
* the logits are the embedding table times the normalised stream.

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v`` (each with ``.b``), ``l<i>.mix.o|lq1|lk1|lq2|lk2``,
``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down``,
``l<i>.hc1|hc2.in|out|mix``, ``final.norm``; matrices are stored ``[out, in]``.
"""

from __future__ import annotations

import math

import torch

from ..config.nodopel_config import DenseMlpConfig, NodopelConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(config: NodopelConfig, name: str) -> PartSpec:
    # The tensor is the norm's own name (no ".weight" behind it).
    return PartSpec("rms_norm", {"eps": config.norm_eps, "weight_name": ""}, name=name)


def _position(config: NodopelConfig, index: int) -> PartSpec:
    rot = config.layers[index].mixer.rot
    if rot is None:
        return PartSpec("none")
    return PartSpec("rotary", {"theta": rot.base, "rotary_dim": rot.dims, "frequency_scaling": rot.scaling})


def _mixer(config: NodopelConfig, index: int) -> PartSpec:
    mixer = config.layers[index].mixer
    return PartSpec("differential_attention", {
        "num_heads": mixer.heads, "num_kv_heads": mixer.kv_heads, "head_dim": mixer.dim, "value_dim": mixer.vdim,
        "scale": mixer.scale, "softcap": mixer.softcap, "window": mixer.window, "keep_first": mixer.keep_first,
        "diff": mixer.diff, "norm_eps": config.norm_eps, "bias": True}, name="mix")


def _feed_forward(mlp) -> PartSpec:
    if isinstance(mlp, DenseMlpConfig):
        return PartSpec("gated_silu", {"intermediate_size": mlp.ff, "activation": "gelu_tanh",
                                       "weight_names": ("gate", "up", "down")}, name="mlp")
    return PartSpec("routed_experts", {
        "num_experts": mlp.experts, "identity_experts": mlp.identity, "top": mlp.top, "intermediate_size": mlp.ff,
        "scoring": "softmax", "renormalise": True, "correction": True,
        "shared_intermediate_size": mlp.shared_ff}, name="mlp")


def build_spec(config: NodopelConfig) -> ModelSpec:
    layers = []
    block = (PartSpec("pre_norm") if config.streams is None
             else PartSpec("hyper_connections", {"streams": config.streams, "names": ("hc1", "hc2")}))
    for index, layer in enumerate(config.layers):
        norms = {"mixer": _norm(config, "norm1")}
        feed_forward = None
        if layer.mlp is not None:
            norms["feed_forward"] = _norm(config, "norm2")
            feed_forward = _feed_forward(layer.mlp)
        layers.append(LayerSpec(name=f"l{index}", block=block, mixer=_mixer(config, index), feed_forward=feed_forward,
                                position=_position(config, index), norms=norms))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("token_embedding", {"weight_name": "embed"}, name=""),
        layers=tuple(layers),
        # a layer of the loop appears once per run: the same weights, a cache of its own each time
        schedule=tuple(ScheduleEntry(layer=index) for index in config.layer_order()),
        final_norm=_norm(config, "final.norm"),
        output_head=PartSpec("linear_head", {"tied": True}, name="head"),
        streams=config.streams,
    )


def random_weights(config: NodopelConfig, seed: int, *, std: float | None = None, norm_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu"
                   ) -> dict[str, torch.Tensor]:
    """Seeded random tensors under the checkpoint's names: matrices ``N(0, std)`` (``std`` defaults to ``fan_in **
    -0.5``, which keeps activations of order one through any width), norm weights ``1 + N(0, norm_std)``, biases
    and the vectors of lambda ``N(0, 0.1)``, the router's correction ``N(0, 0.02)``; the streams' tables near a
    plain residual (``in`` around ``1 / streams``, ``mix`` around the identity, ``out`` around 1), so that a deep
    stack stays of order one."""
    generator = torch.Generator(device=device).manual_seed(seed)

    def normal(shape, mean, spread: float) -> torch.Tensor:
        return (mean + torch.empty(shape, dtype=torch.float32, device=device).normal_(
            0.0, 1.0, generator=generator) * spread).to(dtype)

    def matrix(rows: int, cols: int) -> torch.Tensor:
        return normal((rows, cols), 0.0, std if std is not None else 1.0 / math.sqrt(cols))

    hidden = config.hidden_size
    weights = {"embed": normal((config.vocab_size, hidden), 0.0, 1.0)}
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        mixer = layer.mixer
        weights[p + "norm1"] = normal((hidden,), 1.0, norm_std)
        for name, rows in (("q", mixer.heads * 2 * mixer.dim), ("k", mixer.kv_heads * 2 * mixer.dim),
                           ("v", mixer.kv_heads * mixer.vdim)):
            weights[p + "mix." + name] = matrix(rows, hidden)
            weights[p + "mix." + name + ".b"] = normal((rows,), 0.0, 0.1)
        weights[p + "mix.o"] = matrix(hidden, mixer.heads * mixer.vdim)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            weights[p + "mix." + name] = normal((mixer.dim,), 0.0, 0.1)
        mlp = layer.mlp
        if mlp is not None:
            weights[p + "norm2"] = normal((hidden,), 1.0, norm_std)
            if isinstance(mlp, DenseMlpConfig):
                weights[p + "mlp.gate"] = matrix(mlp.ff, hidden)
                weights[p + "mlp.up"] = matrix(mlp.ff, hidden)
                weights[p + "mlp.down"] = matrix(hidden, mlp.ff)
            else:
                outputs = mlp.experts + mlp.identity
                weights[p + "mlp.router"] = matrix(outputs, hidden)
                weights[p + "mlp.correction"] = normal((outputs,), 0.0, 0.02)
                names = [f"e{expert}" for expert in range(mlp.experts)]
                for name, ff in [(name, mlp.ff) for name in names] + ([("shared", mlp.shared_ff)] if mlp.shared_ff else []):
                    weights[p + f"mlp.{name}.gate"] = matrix(ff, hidden)
                    weights[p + f"mlp.{name}.up"] = matrix(ff, hidden)
                    weights[p + f"mlp.{name}.down"] = matrix(hidden, ff)
        if config.streams is not None:
            count = config.streams
            for name in ("hc1", "hc2")[:1 if mlp is None else 2]:
                weights[p + name + ".in"] = normal((count,), 1.0 / count, 0.1 / count)
                weights[p + name + ".out"] = normal((count,), 1.0, 0.1)
                weights[p + name + ".mix"] = normal((count, count), torch.eye(count, device=device), 0.05)
    weights["final.norm"] = normal((hidden,), 1.0, norm_std)
    return weights


register_architecture("Nodopel", NodopelConfig, build_spec, random_weights)
