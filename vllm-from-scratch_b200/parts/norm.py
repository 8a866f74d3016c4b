"""RMSNorm with the residual sum fused in.

``y = x * rsqrt(mean(x^2) + eps) * weight`` with the statistics in float32
(minivllm/layers/ops/layernorm.py:196-227; class minivllm/layers/layernorm.py:26-52).
The residual stream it adds into is float32.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import NORMS, FreshStreams, Norm, NormedAddend, PartEnv, StreamAddend, WeightInfo


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """params: ``eps`` (inside the root), ``size`` (defaults to the residual width), ``offset``
    (default 0: the checkpoint's vector is the weight; 1 for a vector stored around zero, the weight
    being ``1 + w``), ``weight_name`` (the tensor's name under the part's prefix, default ``weight``;
    empty: the prefix itself is the tensor).

    ``forward`` also takes a :class:`~.base.NormedAddend` for ``x``: rows that pass through a norm of
    their own on their way into the residual; both norms and the sum are then one kernel.  Where the
    residual is kept as several streams (``[T, S, H]``), ``x`` is a :class:`~.base.StreamAddend` (or
    :class:`~.base.FreshStreams`) and the norm reads the plain sum of the updated streams."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.eps = float(params["eps"])
        self.size = int(params.get("size", env.hidden_size))
        self.offset = float(params.get("offset", 0.0))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        return {self.weight_name: WeightInfo((self.size,), "vector")}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()      # float32: formed once, as the norm would

    def addend(self, rows: torch.Tensor) -> NormedAddend:
        """``rows`` on their way into the residual through this norm."""
        return NormedAddend(rows, self.weight, self.eps)

    def split(self) -> tuple[torch.Tensor, float] | None:
        return (self.weight, self.eps) if self.size == self.env.hidden_size else None

    def forward(self, x: torch.Tensor | NormedAddend | None, residual: torch.Tensor, out: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            count = residual.shape[0] if rows is None else rows.shape[0]
            out = torch.empty((count, self.size), dtype=self.env.dtype, device=residual.device)
        if isinstance(x, (StreamAddend, FreshStreams)):
            from ..kernels import streams
            update = ({"fresh": x.rows} if isinstance(x, FreshStreams)
                      else {"rows_in": x.rows, "mix": x.mix, "out_weights": x.out})
            streams.stream_mix_norm(residual, **update, norm_weight=self.weight, eps=self.eps, normed=out, rows=rows)
        elif isinstance(x, NormedAddend):
            kernels.add_normed_rmsnorm(x.rows, x.weight, x.eps, residual, self.weight, self.eps, out, rows)
        else:
            kernels.add_rmsnorm(x, residual, self.weight, self.eps, out, rows)
        return out
