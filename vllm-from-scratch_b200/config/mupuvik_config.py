"""Typed configuration of the Mupuvik decoder, read from its config.json.

The file names the design under ``architecture`` and gives every size and every constant that may
differ between two models of the design: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``) and ``layers``, a list whose entries give a
layer's ``type`` (which mixer: ``attention``, ``parallel`` or ``mamba2``), the mixer's sizes (``mixer``)
and its feed-forward (``mlp``: ``kind`` moe with ``expert`` (``ff``, ``limit``), ``router`` (``experts``,
``top``) and, where it has one, ``shared`` (``ff``, ``limit``); or null).  The rank of the decay's two
small matrices in the gated linear branch is in no key: it is the shape of the tensors.  What the
design fixes (the arrangement of the norms, the forms of the activations, which norm goes where) is
code, in ``models/mupuvik.py`` and the parts it names.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .bemuzen_config import Mamba2MixerConfig, _float, _int, _keys
from .lobuzen_config import _mask, _window
from .model_config import ConfigError


def _heads(where: str, raw: Mapping[str, Any]) -> tuple[int, int]:
    heads, kv_heads = _int(where + ".heads", raw["heads"]), _int(where + ".kv_heads", raw["kv_heads"])
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads


@dataclass(frozen=True)
class WindowedAttentionConfig:
    """The mixer ``attention``: biased projections, a norm over all of q and of k, a window, a gate per head."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    kv_from: int | None             # the layer whose cached keys and values this one reads, if not its own

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "WindowedAttentionConfig":
        raw = _keys(where, raw, ("heads", "kv_heads", "dim", "vdim", "scale"))
        heads, kv_heads = _heads(where, raw)
        kv_from = raw.get("kv_from")
        return cls(heads, kv_heads, _int(where + ".dim", raw["dim"]), _int(where + ".vdim", raw["vdim"]),
                   _float(where + ".scale", raw["scale"]), _window(where, raw),
                   None if kv_from is None else _int(where + ".kv_from", kv_from, 0))

    def to_dict(self) -> dict[str, Any]:
        made = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, **_mask(self.window)}
        if self.kv_from is not None:
            made["kv_from"] = self.kv_from
        return made


@dataclass(frozen=True)
class RotarySinkBranchConfig:
    """Left side of ``parallel``: norm per head, rotated neighbours, causal, one added to the softmax denominator."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float | None          # None: nothing is rotated
    rot_dims: int

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "RotarySinkBranchConfig":
        raw = _keys(where, raw, ("heads", "kv_heads", "dim", "vdim", "scale"))
        heads, kv_heads = _heads(where, raw)
        dim = _int(where + ".dim", raw["dim"])
        base, dims = None, 0
        if raw.get("rot") is not None:
            rot = _keys(where + ".rot", raw["rot"], ("base", "dims"))
            base, dims = _float(where + ".rot.base", rot["base"]), _int(where + ".rot.dims", rot["dims"], 0)
            if base <= 0 or dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}.rot: base={base}, dims={dims} (even, at most dim={dim})")
            if dims == 0:
                base = None
        return cls(heads, kv_heads, dim, _int(where + ".vdim", raw["vdim"]), _float(where + ".scale", raw["scale"]),
                   base, dims)

    def to_dict(self) -> dict[str, Any]:
        made = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_base is not None:
            made["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return made


@dataclass(frozen=True)
class GatedLinearBranchConfig:
    """Right side of ``parallel``: linear attention whose state decays per key channel."""

    heads: int
    dim: int
    vdim: int
    tau: float

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "GatedLinearBranchConfig":
        raw = _keys(where, raw, ("heads", "dim", "vdim", "tau"))
        tau = _float(where + ".tau", raw["tau"])
        if tau <= 0:
            raise ConfigError(f"config.json: {where}.tau must be positive, got {tau}")
        return cls(_int(where + ".heads", raw["heads"]), _int(where + ".dim", raw["dim"]),
                   _int(where + ".vdim", raw["vdim"]), tau)

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: RotarySinkBranchConfig
    right: GatedLinearBranchConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "ParallelMixerConfig":
        raw = _keys(where, raw, ("left", "right", "left_scale", "right_scale"))
        return cls(RotarySinkBranchConfig.from_dict(where + ".left", raw["left"]),
                   GatedLinearBranchConfig.from_dict(where + ".right", raw["right"]),
                   _float(where + ".left_scale", raw["left_scale"]), _float(where + ".right_scale", raw["right_scale"]))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int | None           # None: no expert that every token passes
    shared_limit: float

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "ExpertsConfig":
        raw = _keys(where, raw, ("kind", "expert", "router"))
        if raw["kind"] != "moe":
            raise ConfigError(f"config.json: {where}.kind {raw['kind']!r}: only 'moe' is part of the design")
        expert = _keys(where + ".expert", raw["expert"], ("ff", "limit"))
        router = _keys(where + ".router", raw["router"], ("experts", "top"))
        experts, top = _int(where + ".router.experts", router["experts"]), _int(where + ".router.top", router["top"])
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top ({top}) exceeds experts ({experts})")
        shared_ff, shared_limit = None, 0.0
        if raw.get("shared") is not None:
            shared = _keys(where + ".shared", raw["shared"], ("ff", "limit"))
            shared_ff, shared_limit = _int(where + ".shared.ff", shared["ff"]), _float(where + ".shared.limit", shared["limit"])
        return cls(experts, top, _int(where + ".expert.ff", expert["ff"]), _float(where + ".expert.limit", expert["limit"]),
                   shared_ff, shared_limit)

    def to_dict(self) -> dict[str, Any]:
        made = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            made["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return made


_MIXERS = {"attention": WindowedAttentionConfig, "parallel": ParallelMixerConfig, "mamba2": Mamba2MixerConfig}


@dataclass(frozen=True)
class MupuvikLayerConfig:
    type: str
    mixer: WindowedAttentionConfig | ParallelMixerConfig | Mamba2MixerConfig
    mlp: ExpertsConfig | None       # None: the layer has no feed-forward

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "MupuvikLayerConfig":
        raw = _keys(where, raw, ("type", "mixer"))
        kind = raw["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                              f"({', '.join(sorted(_MIXERS))})")
        mlp = raw.get("mlp")
        return cls(kind, _MIXERS[kind].from_dict(where + ".mixer", raw["mixer"]),
                   None if mlp is None else ExpertsConfig.from_dict(where + ".mlp", mlp))

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class MupuvikConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[MupuvikLayerConfig, ...]
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MupuvikConfig":
        raw = _keys("the file", raw, ("architecture", "vocab", "width", "norm", "embedding", "layers"))
        norm = _keys("norm", raw["norm"], ("eps",))
        embedding = _keys("embedding", raw["embedding"], ("scale", "bigram"))
        bigram = _keys("embedding.bigram", embedding["bigram"], ("buckets", "mul_prev", "mul_cur"))
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        eps = _float("norm.eps", norm["eps"])
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        made = tuple(MupuvikLayerConfig.from_dict(f"layers[{index}]", layer) for index, layer in enumerate(layers))
        for index, layer in enumerate(made):
            source = getattr(layer.mixer, "kv_from", None)
            if source is None:
                continue
            owner = made[source].mixer if source < index else None
            if not isinstance(owner, WindowedAttentionConfig) or owner.kv_from is not None:
                raise ConfigError(f"config.json: layers[{index}].mixer.kv_from={source} must name an earlier attention "
                                  f"layer that has keys and values of its own")
            if (owner.kv_heads, owner.dim, owner.vdim) != (layer.mixer.kv_heads, layer.mixer.dim, layer.mixer.vdim):
                raise ConfigError(f"config.json: layers[{index}] reads the keys and values of layers[{source}], whose "
                                  f"kv_heads, dim and vdim differ from its own")
        return cls(
            architecture=str(raw["architecture"]), vocab_size=_int("vocab", raw["vocab"]),
            hidden_size=_int("width", raw["width"]), norm_eps=eps,
            embedding_scale=_float("embedding.scale", embedding["scale"]),
            bigram_buckets=_int("embedding.bigram.buckets", bigram["buckets"]),
            bigram_mul_prev=_int("embedding.bigram.mul_prev", bigram["mul_prev"], 0),
            bigram_mul_cur=_int("embedding.bigram.mul_cur", bigram["mul_cur"], 0),
            layers=made, initializer_range=float(raw.get("initializer_range", 0.05)))

    @classmethod
    def from_json(cls, path: str | Path) -> "MupuvikConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def to_dict(self) -> dict[str, Any]:
        """config.json content that reads back to an equal object."""
        return {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "embedding": {"scale": self.embedding_scale,
                          "bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                     "mul_cur": self.bigram_mul_cur}},
            "layers": [layer.to_dict() for layer in self.layers],
            "initializer_range": self.initializer_range,
        }

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def summary(self) -> list[str]:
        """A few lines that describe the model to a reader of the command line's output."""
        kinds = [layer.type + ("" if layer.mlp is not None else " (no feed-forward)") for layer in self.layers]
        runs: list[list] = []
        for kind in kinds:
            if runs and runs[-1][0] == kind:
                runs[-1][1] += 1
            else:
                runs.append([kind, 1])
        return [f"{len(self.layers)} layers, width={self.hidden_size}, vocabulary={self.vocab_size}, "
                f"bigram buckets={self.bigram_buckets}",
                "order of layers: " + ", ".join(f"{count} x {kind}" for kind, count in runs)]
