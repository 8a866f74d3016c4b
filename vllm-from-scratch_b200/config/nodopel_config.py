"""Typed configuration of the Nodopel decoder, read from its config.json.

The file names the design under ``architecture`` and gives every size and every constant that may
differ between two models of the design: ``vocab``, ``width``, ``norm.eps``, ``streams`` (how many copies
of the residual stream the hyper-connections keep; absent: a plain residual), ``loop`` (``start``,
``stop``, ``times``: the layers that run several times in a row with the same weights) and ``layers``, a
list whose entries give a layer's ``type`` (which mixer), the mixer's sizes and constants (``mixer``) and
its feed-forward (``mlp``: ``kind`` dense with ``ff``, or ``kind`` moe with ``expert.ff``, ``router`` and an
optional ``shared.ff``; or null).  What the design fixes (the pre-norm arrangement, two maps to a head, the
activations, a softmax router whose weights are renormalised) is code, in ``models/nodopel.py`` and the
parts it names.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .bemuzen_config import _float, _int, _keys
from .model_config import ConfigError


@dataclass(frozen=True)
class RotationConfig:
    dims: int                       # channels of every map of every head that are rotated
    base: float
    # Stretching of long wavelengths: (factor, low, high, original), or None.
    scaling: tuple[float, float, float, int] | None

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "RotationConfig | None":
        if raw is None:
            return None
        raw = _keys(where, raw, ("dims", "base"))
        dims = _int(where + ".dims", raw["dims"], 2)
        if dims % 2:
            raise ConfigError(f"config.json: {where}.dims ({dims}) must be even")
        base = _float(where + ".base", raw["base"])
        if base <= 0:
            raise ConfigError(f"config.json: {where}.base must be positive, got {base}")
        scaling = raw.get("scaling")
        if scaling is not None:
            s = _keys(where + ".scaling", scaling, ("factor", "low", "high", "original"))
            scaling = (_float(where + ".scaling.factor", s["factor"]), _float(where + ".scaling.low", s["low"]),
                       _float(where + ".scaling.high", s["high"]), _int(where + ".scaling.original", s["original"]))
            if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= scaling[1]:
                raise ConfigError(f"config.json: {where}.scaling wants factor > 0 and high > low > 0, got {s!r}")
        return cls(dims, base, scaling)

    def to_dict(self) -> dict[str, Any]:
        made: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            factor, low, high, original = self.scaling
            made["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
        return made


@dataclass(frozen=True)
class DifferentialMixerConfig:
    heads: int
    kv_heads: int
    dim: int                        # of one map's queries and keys
    vdim: int
    scale: float
    diff: float                     # the constant in lambda and in the output's factor 1 - diff
    softcap: float | None
    window: int | None              # positions a query sees behind itself (itself included); None: all
    keep_first: int                 # positions at the start of a sequence that stay visible whatever the window
    rot: RotationConfig | None

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "DifferentialMixerConfig":
        raw = _keys(where, raw, ("heads", "kv_heads", "dim", "vdim", "scale", "diff"))
        heads, kv_heads = _int(where + ".heads", raw["heads"]), _int(where + ".kv_heads", raw["kv_heads"])
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        softcap = raw.get("softcap")
        if softcap is not None:
            softcap = _float(where + ".softcap", softcap)
            if softcap <= 0:
                raise ConfigError(f"config.json: {where}.softcap must be positive, got {softcap}")
        window, keep_first = None, 0
        mask = raw.get("mask")
        if mask is not None:
            mask = _keys(where + ".mask", mask, ())
            if mask.get("size") is not None:
                window = _int(where + ".mask.size", mask["size"])
            if mask.get("keep_first") is not None:
                keep_first = _int(where + ".mask.keep_first", mask["keep_first"], 0)
        dim = _int(where + ".dim", raw["dim"])
        rot = RotationConfig.from_dict(where + ".rot", raw.get("rot"))
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims ({rot.dims}) exceeds dim ({dim})")
        return cls(heads, kv_heads, dim, _int(where + ".vdim", raw["vdim"]), _float(where + ".scale", raw["scale"]),
                   _float(where + ".diff", raw["diff"]), softcap, window, keep_first if window is not None else 0, rot)

    def to_dict(self) -> dict[str, Any]:
        made: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                                "scale": self.scale, "diff": self.diff}
        if self.softcap is not None:
            made["softcap"] = self.softcap
        if self.window is not None:
            made["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot is not None:
            made["rot"] = self.rot.to_dict()
        return made


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MoeMlpConfig:
    ff: int                         # of one expert
    experts: int                    # experts that have tensors
    identity: int                   # router outputs behind them whose expert is the identity
    top: int
    shared_ff: int | None           # width of the expert that every token passes, if there is one

    def to_dict(self) -> dict[str, Any]:
        made: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}
        if self.shared_ff is not None:
            made["shared"] = {"ff": self.shared_ff}
        return made


def _mlp(where: str, raw: Any) -> DenseMlpConfig | MoeMlpConfig | None:
    if raw is None:
        return None
    raw = _keys(where, raw, ("kind",))
    if raw["kind"] == "dense":
        raw = _keys(where, raw, ("ff",))
        return DenseMlpConfig(_int(where + ".ff", raw["ff"]))
    if raw["kind"] == "moe":
        raw = _keys(where, raw, ("expert", "router"))
        expert = _keys(where + ".expert", raw["expert"], ("ff",))
        router = _keys(where + ".router", raw["router"], ("experts", "top"))
        experts, top = _int(where + ".router.experts", router["experts"]), _int(where + ".router.top", router["top"])
        identity = 0 if router.get("identity") is None else _int(where + ".router.identity", router["identity"], 0)
        if top > experts + identity:
            raise ConfigError(f"config.json: {where}.router: top={top} of {experts} + {identity} experts")
        shared = raw.get("shared")
        shared_ff = None
        if shared is not None:
            shared_ff = _int(where + ".shared.ff", _keys(where + ".shared", shared, ("ff",))["ff"])
        return MoeMlpConfig(_int(where + ".expert.ff", expert["ff"]), experts, identity, top, shared_ff)
    raise ConfigError(f"config.json: {where}.kind {raw['kind']!r}: 'dense' and 'moe' are part of the design")


_MIXERS = {"attention": DifferentialMixerConfig}


@dataclass(frozen=True)
class NodopelLayerConfig:
    type: str
    mixer: DifferentialMixerConfig
    mlp: DenseMlpConfig | MoeMlpConfig | None

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "NodopelLayerConfig":
        raw = _keys(where, raw, ("type", "mixer"))
        kind = raw["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                              f"({', '.join(sorted(_MIXERS))})")
        return cls(kind, _MIXERS[kind].from_dict(where + ".mixer", raw["mixer"]), _mlp(where + ".mlp", raw.get("mlp")))

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class NodopelConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    streams: int | None             # None: one residual stream and plain sums
    loop: tuple[int, int, int] | None       # (start, stop, times)
    layers: tuple[NodopelLayerConfig, ...]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NodopelConfig":
        raw = _keys("the file", raw, ("architecture", "vocab", "width", "norm", "layers"))
        norm = _keys("norm", raw["norm"], ("eps",))
        eps = _float("norm.eps", norm["eps"])
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        streams = None if raw.get("streams") is None else _int("streams", raw["streams"])
        loop = raw.get("loop")
        if loop is not None:
            loop = _keys("loop", loop, ("start", "stop", "times"))
            loop = (_int("loop.start", loop["start"], 0), _int("loop.stop", loop["stop"], 0), _int("loop.times", loop["times"]))
            if not loop[0] <= loop[1] <= len(layers):
                raise ConfigError(f"config.json: loop {loop[0]} .. {loop[1]} does not lie within the {len(layers)} layers")
        return cls(str(raw["architecture"]), _int("vocab", raw["vocab"]), _int("width", raw["width"]), eps, streams, loop,
                   tuple(NodopelLayerConfig.from_dict(f"layers[{index}]", layer) for index, layer in enumerate(layers)))

    @classmethod
    def from_json(cls, path: str | Path) -> "NodopelConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def to_dict(self) -> dict[str, Any]:
        """config.json content that reads back to an equal object."""
        made: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                                "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.streams is not None:
            made["streams"] = self.streams
        if self.loop is not None:
            made["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return made

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def layer_order(self) -> list[int]:
        """The layers' numbers in the order they run: those of the loop ``times`` times in a row."""
        count = len(self.layers)
        if self.loop is None:
            return list(range(count))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))

    def summary(self) -> list[str]:
        """A few lines that describe the model to a reader of the command line's output."""
        def kind(layer: NodopelLayerConfig) -> str:
            mlp = "no feed-forward" if layer.mlp is None else "dense" if isinstance(layer.mlp, DenseMlpConfig) else "experts"
            return f"{layer.type} ({mlp})"
        runs: list[list] = []
        for name in (kind(self.layers[index]) for index in self.layer_order()):
            if runs and runs[-1][0] == name:
                runs[-1][1] += 1
            else:
                runs.append([name, 1])
        return [f"{len(self.layers)} layers in {len(self.layer_order())} runs, width={self.hidden_size}, "
                f"vocabulary={self.vocab_size}, streams={'one' if self.streams is None else self.streams}",
                "order of runs: " + ", ".join(f"{count} x {name}" for name, count in runs)]
