"""Two mixers side by side on the same input.  ``combine="norm_mean"`` (the default): ``(rms(left(h)) * w_left +
rms(right(h)) * w_right) / 2``, each branch's output normalised over the model width with a plain weight vector
of its own before the mean.  ``combine="weighted_sum"``: ``scales[0] * left(h) + scales[1] * right(h)``, nothing
else; where both branches end in an output product and can hand over what it multiplies (``forward_inner``,
``inner_width``, ``out_proj``), the sum is one product: the branches write their rows, each times its scale, side by
side, and ``[W_left | W_right]`` multiplies them.  The branches are mixers of any registered kind, built from their own :class:`~.spec.PartSpec`;
their tensors live under the names the specs give (``left`` and ``right`` by default), their cache
needs are handed on together (at most one of them may keep pages), and each finds its share of the
layer's :class:`~.base.CacheView`.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import (MIXERS, CacheView, KVPagesNeed, Mixer, PartEnv, PositionEncoding, StateNeed, StepContext,
                   WeightInfo)
from .spec import PartSpec


def _join(prefix: str, name: str) -> str:
    return f"{prefix}.{name}" if prefix and name else prefix or name


@MIXERS.register("paired_mixers")
class PairedMixers(Mixer):
    """params: ``branches`` (two :class:`~.spec.PartSpec` of mixers; each spec's ``name`` is the segment
    of its tensors and of its output norm vector ``<name>.<out_name>``), ``combine`` (``norm_mean`` or
    ``weighted_sum``), for the mean ``eps`` and ``out_name`` (default ``out``), for the sum ``scales`` (two
    numbers)."""

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        branches = tuple(params["branches"])
        if len(branches) != 2 or not all(isinstance(branch, PartSpec) for branch in branches):
            raise ValueError("paired mixers take two branches, each the spec of a mixer")
        if not all(branch.name for branch in branches) or branches[0].name == branches[1].name:
            raise ValueError("the two branches need names of their own")
        self.combine = str(params.get("combine", "norm_mean"))
        if self.combine not in ("norm_mean", "weighted_sum"):
            raise ValueError(f"paired mixers combine by 'norm_mean' or 'weighted_sum', not {self.combine!r}")
        self.eps = float(params.get("eps", 0.0))
        self.out_name = str(params.get("out_name", "out"))
        self.scales = tuple(float(value) for value in params.get("scales", (1.0, 1.0)))
        if len(self.scales) != 2:
            raise ValueError("paired mixers take one scale for each of the two branches")
        self.specs = branches
        self.branches: list[Mixer] = [
            MIXERS.get(branch.kind)(branch.params, PartEnv(env.hidden_size, env.dtype, env.device,
                                                           _join(env.prefix, branch.name)), position)
            for branch in branches]
        self.out_weights: list[torch.Tensor | None] = [None, None]
        self.joined_out: torch.Tensor | None = None

    @property
    def graph_safe(self) -> bool:       # a pair may be replayed if both branches may
        return all(branch.graph_safe for branch in self.branches)

    def expected_weights(self) -> dict[str, WeightInfo]:
        names: dict[str, WeightInfo] = {}
        for spec, branch in zip(self.specs, self.branches):
            for name, info in branch.expected_weights().items():
                names[_join(spec.name, name)] = info
            if self.combine == "norm_mean":
                names[_join(spec.name, self.out_name)] = WeightInfo((self.env.hidden_size,), "vector")
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for index, (spec, branch) in enumerate(zip(self.specs, self.branches)):
            branch.load_weights({name: tensors[_join(spec.name, name)] for name in branch.expected_weights()})
            if self.combine == "norm_mean":
                self.out_weights[index] = tensors[_join(spec.name, self.out_name)]
        if self.combine == "weighted_sum" and all(
                hasattr(branch, "forward_inner") and getattr(branch, "out_proj", None) is not None
                for branch in self.branches):
            self.joined_out = torch.cat([branch.out_proj for branch in self.branches], dim=1).contiguous()
            for branch in self.branches:
                branch.out_proj = None          # held once, in the joined matrix

    # -------------------------------------------------------------------- cache
    def _needs(self) -> list[list]:
        found = []
        for branch in self.branches:
            need = branch.cache_need()
            found.append([] if need is None else list(need) if isinstance(need, (tuple, list)) else [need])
        return found

    def cache_need(self) -> tuple | None:
        merged: list = []
        for spec, needs in zip(self.specs, self._needs()):
            for need in needs:
                if isinstance(need, StateNeed):
                    need = StateNeed(need.shape, need.dtype, name=_join(spec.name, need.name))
                merged.append(need)
        if sum(isinstance(need, KVPagesNeed) for need in merged) > 1:
            raise ValueError("only one of two paired mixers may keep pages of keys and values")
        return tuple(merged) or None

    def _view(self, index: int, cache: CacheView) -> CacheView:
        """The branch's share of the layer's cache, under the names the branch gave."""
        needs = self._needs()[index]
        prefix = self.specs[index].name + "."
        states = {name[len(prefix):]: tensor for name, tensor in cache.states.items() if name.startswith(prefix)}
        first = next(iter(states.values()), None)
        if any(isinstance(need, KVPagesNeed) for need in needs):
            return CacheView("pages", cache.group, cache.keys, cache.values, first, cache.writable, states)
        if states:
            return CacheView("state", state=first, writable=cache.writable, states=states)
        return CacheView("none")

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if self.joined_out is not None:
            widths = [branch.inner_width() for branch in self.branches]
            rows = torch.empty((x.shape[0], sum(widths)), dtype=x.dtype, device=x.device)
            self.branches[0].forward_inner(x, ctx, self._view(0, cache), self.scales[0], rows[:, :widths[0]])
            self.branches[1].forward_inner(x, ctx, self._view(1, cache), self.scales[1], rows[:, widths[0]:])
            out = torch.empty((x.shape[0], self.env.hidden_size), dtype=x.dtype, device=x.device)
            kernels.gemm(rows, self.joined_out, out)
            return out
        left = self.branches[0].forward(x, ctx, self._view(0, cache))
        right = self.branches[1].forward(x, ctx, self._view(1, cache))
        out = torch.empty_like(left)
        if self.combine == "weighted_sum":
            kernels.scaled_sum(left, self.scales[0], right, self.scales[1], out)
        else:
            kernels.paired_norm_mean(left, self.out_weights[0], right, self.out_weights[1], self.eps, out)
        return out
