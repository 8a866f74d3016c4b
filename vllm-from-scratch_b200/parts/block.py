"""Arrangement of a layer's parts around the residual stream.

``pre_norm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))``, written with
the not-yet-added output carried beside the residual so that every addition is
fused into the next norm (minivllm/models/qwen3.py:216-233).

For steps of a few tokens, where the mixer and the feed-forward say that they split norms
(:meth:`~.base.Mixer.splits_norms`), neither norm runs as a kernel of its own: the product
ahead of a norm adds into the residual and hands on :class:`~.base.HalfNormedRows`, the
product behind it applies the root; the second product of the feed-forward does so under
the next block's first norm."""

from __future__ import annotations

import torch

from .. import kernels
from .base import (BLOCKS, Block, CacheView, FreshStreams, HalfNormedRows, Norm, NormedAddend,  # noqa: F401
                   StepContext, StreamAddend, WeightInfo)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h += mixer(norm1(h)); h += feed_forward(norm2(h))``; a layer without a feed-forward is its first half."""

    norm_roles = ("mixer", "feed_forward")
    graph_safe = True
    needs_feed_forward = False

    def __init__(self, params, env, *, mixer, feed_forward, norms, side=None) -> None:
        self.norm_roles = ("mixer", "feed_forward") if feed_forward is not None else ("mixer",)
        super().__init__(params, env, mixer=mixer, feed_forward=feed_forward, norms=norms, side=side)

    def _splits_norms(self, tokens: int) -> bool:
        return (self.feed_forward is not None and self.norms["feed_forward"].split() is not None
                and self.mixer.splits_norms(tokens) and self.feed_forward.splits_norms(tokens))

    def first_norm(self) -> Norm:
        return self.norms["mixer"]

    def takes_half_normed(self, tokens: int) -> bool:
        return self.norms["mixer"].split() is not None and self._splits_norms(tokens)

    def folds_into(self, norm: Norm, tokens: int) -> bool:
        return norm.split() is not None and self._splits_norms(tokens)

    def forward(self, x: torch.Tensor | HalfNormedRows | None, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView, next_norm: Norm | None = None) -> torch.Tensor | HalfNormedRows:
        normed = x if isinstance(x, HalfNormedRows) else self.norms["mixer"].forward(x, residual)
        if not self._splits_norms(residual.shape[0]):
            mixed = self.mixer.forward(normed, ctx, cache)
            if self.feed_forward is None:
                return mixed
            normed = self.norms["feed_forward"].forward(mixed, residual)
            return self.feed_forward.forward(normed, ctx)
        half = self.mixer.forward(normed, ctx, cache, fold=(residual, self.norms["feed_forward"]))
        return self.feed_forward.forward(half, ctx, fold=None if next_norm is None else (residual, next_norm))


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm in front of and behind each sublayer: ``h += post_mixer(mixer(mixer_norm(h)))``, then,
    where the layer has a feed-forward, ``h += post_feed_forward(feed_forward(feed_forward_norm(h)))``.

    What a sublayer returns travels on as a :class:`~.base.NormedAddend` under the norm behind it, so
    that norm, the sum into the residual and the norm in front of the next sublayer (the next layer's,
    or the model's last one) are one kernel."""

    graph_safe = True
    needs_feed_forward = False

    def __init__(self, params, env, *, mixer, feed_forward, norms) -> None:
        self.norm_roles = (("mixer", "post_mixer", "feed_forward", "post_feed_forward") if feed_forward is not None
                           else ("mixer", "post_mixer"))
        super().__init__(params, env, mixer=mixer, feed_forward=feed_forward, norms=norms)
        for role, norm in self.norms.items():
            if role.startswith("post_") and not hasattr(norm, "addend"):
                raise ValueError(f"block at {env.prefix!r}: the norm behind a sublayer ({role}) must be able to "
                                 f"travel with its rows (an `addend` method)")

    def forward(self, x, residual: torch.Tensor, ctx: StepContext, cache: CacheView):
        normed = self.norms["mixer"].forward(x, residual)
        mixed = self.norms["post_mixer"].addend(self.mixer.forward(normed, ctx, cache))
        if self.feed_forward is None:
            return mixed
        normed = self.norms["feed_forward"].forward(mixed, residual)
        return self.norms["post_feed_forward"].addend(self.feed_forward.forward(normed, ctx))


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    """A norm behind each sublayer and none in front: ``h += post_mixer(mixer(h))``, then, where the layer
    has one, ``h += post_feed_forward(feed_forward(h))``, then, where the layer has one, ``h +=
    post_side(side(h, tokens))``.  Every sublayer reads the residual stream itself (in the run dtype).

    What a sublayer returns travels on as a :class:`~.base.NormedAddend`; the kernel that normalises it and
    adds it into the float32 residual also writes the sum in the run dtype, which the next sublayer (the next
    layer's mixer) reads.  In the float32 run mode the sublayers read the residual in place."""

    graph_safe = True
    needs_feed_forward = False
    takes_side = True

    def __init__(self, params, env, *, mixer, feed_forward, norms, side=None) -> None:
        roles = ["post_mixer"]
        if feed_forward is not None:
            roles.append("post_feed_forward")
        if side is not None:
            roles.append("post_side")
        self.norm_roles = tuple(roles)
        super().__init__(params, env, mixer=mixer, feed_forward=feed_forward, norms=norms, side=side)
        for role, norm in self.norms.items():
            if not hasattr(norm, "addend"):
                raise ValueError(f"block at {env.prefix!r}: the norm behind a sublayer ({role}) must be able to "
                                 f"travel with its rows (an `addend` method)")

    def _rows(self, pending: NormedAddend | None, residual: torch.Tensor) -> torch.Tensor:
        """Add what is pending into the residual and return the stream as the next sublayer reads it."""
        if pending is not None and not isinstance(pending, NormedAddend):
            raise ValueError("a post-norm block takes what is handed to it as rows under the norm behind them")
        addend = (None, None, 0.0) if pending is None else (pending.rows, pending.weight, pending.eps)
        if self.env.dtype == torch.float32:
            if pending is not None:
                kernels.add_normed_rmsnorm(*addend, residual, None, 0.0, None)
            return residual
        rows = torch.empty(residual.shape, dtype=self.env.dtype, device=residual.device)
        kernels.add_normed_rmsnorm(*addend, residual, None, 0.0, rows)
        return rows

    def forward(self, x, residual: torch.Tensor, ctx: StepContext, cache: CacheView) -> NormedAddend:
        pending = self.norms["post_mixer"].addend(self.mixer.forward(self._rows(x, residual), ctx, cache))
        if self.feed_forward is not None:
            rows = self._rows(pending, residual)
            pending = self.norms["post_feed_forward"].addend(self.feed_forward.forward(rows, ctx))
        if self.side is not None:
            rows = self._rows(pending, residual)
            pending = self.norms["post_side"].addend(self.side.forward(rows, ctx))
        return pending


@BLOCKS.register("hyper_connections")
class HyperConnectionBlock(Block):
    """The pre-norm arrangement over a residual that is kept as ``streams`` copies ``X_1 .. X_S`` (float32 ``[T,
    S, H]``, all equal to the embedding's rows at the start of the model).  For sublayer q (1: the mixer, 2: the
    feed-forward) with its tensors ``in`` ``[S]``, ``out`` ``[S]`` and ``mix`` ``[S, S]`` (indexed ``[from, to]``)::

        u = sum_s in[s] X_s;   y = sublayer(norm(u));   X_t <- sum_s mix[s, t] X_s + out[t] y   (all t at once)

    What a sublayer returns travels on as a :class:`~.base.StreamAddend`, so that the update of the streams, the
    weighted sum that the next sublayer reads (the next layer's, or the model's last norm over the plain sum)
    and its RMSNorm are one kernel.  The norms must be plain RMSNorms (a weight and an eps).

    params: ``streams``; ``names`` (the prefixes of the two sublayers' tensors; default ``hc1``, ``hc2``)."""

    norm_roles = ("mixer", "feed_forward")
    graph_safe = True
    needs_feed_forward = False

    def __init__(self, params, env, *, mixer, feed_forward, norms) -> None:
        self.norm_roles = ("mixer", "feed_forward") if feed_forward is not None else ("mixer",)
        super().__init__(params, env, mixer=mixer, feed_forward=feed_forward, norms=norms)
        self.streams = int(params["streams"])
        from ..kernels.streams import MAX_STREAMS
        if not 1 <= self.streams <= MAX_STREAMS:
            raise ValueError(f"block at {env.prefix!r}: streams={self.streams} (1 to {MAX_STREAMS} are built)")
        self.names = tuple(params.get("names", ("hc1", "hc2")))[:len(self.norm_roles)]
        for role, norm in self.norms.items():
            if not hasattr(norm, "weight") or not hasattr(norm, "eps"):
                raise ValueError(f"block at {env.prefix!r}: the norm in front of the {role} must be an RMSNorm")
        self.tables: dict[str, torch.Tensor] = {}

    def expected_weights(self) -> dict[str, WeightInfo]:
        count = self.streams
        names = {}
        for name in self.names:
            names[f"{name}.in"] = WeightInfo((count,), "vector")
            names[f"{name}.out"] = WeightInfo((count,), "vector")
            names[f"{name}.mix"] = WeightInfo((count, count), "vector")
        return names

    def load_weights(self, tensors) -> None:
        self.tables = {name: tensor.contiguous() for name, tensor in tensors.items()}

    def _read(self, pending, residual: torch.Tensor, name: str, norm) -> torch.Tensor:
        """Apply what is pending to the streams, then the weighted sum under ``name`` and its norm."""
        from ..kernels import streams
        if isinstance(pending, FreshStreams):
            update = {"fresh": pending.rows}
        elif isinstance(pending, StreamAddend):
            update = {"rows_in": pending.rows, "mix": pending.mix, "out_weights": pending.out}
        else:
            raise ValueError("a block over several streams takes what is handed to it as rows on their way into "
                             "the streams (StreamAddend) or as the embedding's rows (FreshStreams)")
        normed = torch.empty((residual.shape[0], residual.shape[2]), dtype=self.env.dtype, device=residual.device)
        streams.stream_mix_norm(residual, **update, in_weights=self.tables[f"{name}.in"], norm_weight=norm.weight,
                                eps=norm.eps, normed=normed)
        return normed

    def forward(self, x, residual: torch.Tensor, ctx: StepContext, cache: CacheView) -> StreamAddend:
        if residual.dim() != 3 or residual.shape[1] != self.streams:
            raise ValueError(f"block at {self.env.prefix!r} keeps {self.streams} streams, the residual is "
                             f"{tuple(residual.shape)}")
        first = self.names[0]
        normed = self._read(x, residual, first, self.norms["mixer"])
        pending = StreamAddend(self.mixer.forward(normed, ctx, cache), self.tables[f"{first}.mix"], self.tables[f"{first}.out"])
        if self.feed_forward is None:
            return pending
        second = self.names[1]
        normed = self._read(pending, residual, second, self.norms["feed_forward"])
        return StreamAddend(self.feed_forward.forward(normed, ctx), self.tables[f"{second}.mix"], self.tables[f"{second}.out"])
