"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` (or with the tanh form of gelu on the
gate), no biases (minivllm/models/qwen3.py:44-65).  ``gate`` and ``up`` are held as one matrix
``[2 I, H]`` with the gate rows first (minivllm/layers/linear.py:261-359), so one
product serves both."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import FEED_FORWARDS, FeedForward, HalfNormedRows, Norm, PartEnv, StepContext, WeightInfo


@FEED_FORWARDS.register("gated_silu")
class GatedSiluFeedForward(FeedForward):
    """params: ``intermediate_size``; ``weight_names`` (the checkpoint's names of the gate, up and
    down matrices under the part's prefix; default ``gate_proj.weight``, ``up_proj.weight``,
    ``down_proj.weight``); ``activation`` (of the gate: ``silu``, the default, or ``gelu_tanh``, ``z / 2 * (1
    + tanh(sqrt(2 / pi) * (z + 0.044715 z^3)))``, in float32)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.intermediate_size = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: activation {self.activation!r} ('silu' or 'gelu_tanh')")
        self.names = tuple(params.get("weight_names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.gate_up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        inter, hidden = self.intermediate_size, self.env.hidden_size
        gate, up, down = self.names
        return {gate: WeightInfo((inter, hidden)), up: WeightInfo((inter, hidden)), down: WeightInfo((hidden, inter))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        self.gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()
        self.down = tensors[down].contiguous()

    def splits_norms(self, tokens: int) -> bool:
        return (self.activation == "silu" and kernels.split_norm_ok(tokens, self.gate_up, fold=False, gated=True)
                and kernels.split_norm_ok(tokens, self.down, fold=True))

    def forward(self, x: torch.Tensor | HalfNormedRows, ctx: StepContext,
                fold: tuple[torch.Tensor, Norm] | None = None) -> torch.Tensor | HalfNormedRows:
        scale = (x.squares, x.eps) if isinstance(x, HalfNormedRows) else None
        x = x.rows if isinstance(x, HalfNormedRows) else x
        tokens = x.shape[0]
        hidden = torch.empty((tokens, self.intermediate_size), dtype=x.dtype, device=x.device)
        if self.activation == "silu":
            kernels.gated_silu_gemm(x, self.gate_up, hidden, scale=scale)
        else:
            from ..kernels import grouped
            gate_up = torch.empty((tokens, 2 * self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.gemm(x, self.gate_up, gate_up)
            grouped.gelu_mul(gate_up, hidden)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        if fold is None:
            kernels.gemm(hidden, self.down, out)
            return out
        residual, norm = fold
        weight, eps = norm.split()
        squares = torch.empty((tokens, self.env.hidden_size // 8), dtype=torch.float32, device=x.device)
        kernels.gemm(hidden, self.down, out, fold=(residual, weight, squares))
        return HalfNormedRows(out, squares, eps)


@FEED_FORWARDS.register("capped_gated")
class CappedGatedFeedForward(FeedForward):
    """``down(g * sigmoid(slope * g) * (u + up_offset))`` with ``g = min(gate(x), limit)`` and ``u = clamp(up(x),
    -limit, limit)``; the activation in float32.

    params: ``intermediate_size``, ``limit`` (None: no cap), ``slope`` (default 1.702), ``up_offset`` (default 1),
    ``weight_names`` (gate, up, down; default ``gate``, ``up``, ``down``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.intermediate_size = int(params["intermediate_size"])
        limit = params.get("limit")
        self.limit = None if limit is None else float(limit)
        self.slope = float(params.get("slope", 1.702))
        self.up_offset = float(params.get("up_offset", 1.0))
        self.names = tuple(params.get("weight_names", ("gate", "up", "down")))
        self.gate_up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        inter, hidden = self.intermediate_size, self.env.hidden_size
        gate, up, down = self.names
        return {gate: WeightInfo((inter, hidden)), up: WeightInfo((inter, hidden)), down: WeightInfo((hidden, inter))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        self.gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()
        self.down = tensors[down].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from ..kernels import grouped
        tokens = x.shape[0]
        gate_up = torch.empty((tokens, 2 * self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.gate_up, gate_up)
        hidden = torch.empty((tokens, self.intermediate_size), dtype=x.dtype, device=x.device)
        grouped.capped_swish_mul(gate_up, hidden, self.limit, self.slope, self.up_offset)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(hidden, self.down, out)
        return out


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of small gated feed-forwards, ``down_e(silu(gate_e x) * up_e x)``, of which every token uses
    ``top``: router logits in float32, scores = sigmoid(logits) (``scoring="softmax"``: the softmax over all
    router outputs); the choice is made on ``score + correction``
    (where the checkpoint has a correction), among the experts of the ``group_keep`` best of ``group_count``
    equal groups of neighbouring experts (a group's mark is the sum of its ``group_top`` largest choice
    scores); the output is the sum of the chosen experts' outputs weighted with their plain scores
    (``renormalise``: divided by their sum + 1e-20).  The last ``identity_experts`` router outputs have no
    tensors: their expert's output is its input.  With ``shared_intermediate_size`` an expert of that width,
    of the same form, runs for every token and is added unweighted.  ``activation`` gives the experts another
    form, ``("capped", limit, slope, offset)``: ``down_e(g sigmoid(slope g) (u + offset))`` with ``g = min(gate_e x,
    limit)`` and ``u = clamp(up_e x, -limit, limit)``; the shared expert has constants of its own
    (``shared_activation``).  With ``weight_on_input`` a chosen expert's weight multiplies what it is given, not
    what it returns: the output is the plain sum of ``expert_e(weight_e x)``.

    The tokens of a step are put into one list per expert on the device, the experts' products run as two
    grouped kernels over those lists (the first with the activation in its epilogue), and a last kernel adds
    every token's rows in the order of its choices: nothing depends on host values, whatever the routing.

    params: ``num_experts``, ``top``, ``intermediate_size``, ``group_count`` (default 1), ``group_keep``
    (default ``group_count``), ``group_top`` (default 2), ``correction`` (default True), ``router_name``
    (default ``router``), ``correction_name`` (default ``correction``), ``expert_names`` (patterns with
    ``{index}`` for gate, up, down; default ``e{index}.gate``, ``e{index}.up``, ``e{index}.down``), ``scoring``
    (default ``sigmoid``), ``renormalise`` (default False), ``identity_experts`` (default 0; ``num_experts`` counts
    the experts that have tensors, the router has ``num_experts + identity_experts`` outputs),
    ``shared_intermediate_size`` (default None), ``shared_names`` (gate, up, down; default ``shared.gate``,
    ``shared.up``, ``shared.down``), ``activation`` and ``shared_activation`` (``"silu"``, the default, or
    ``("capped", limit, slope, offset)``), ``weight_on_input`` (default False)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.num_experts = int(params["num_experts"])
        self.top = int(params["top"])
        self.intermediate_size = int(params["intermediate_size"])
        self.group_count = int(params.get("group_count", 1))
        self.group_keep = int(params.get("group_keep", self.group_count))
        self.group_top = int(params.get("group_top", 2))
        self.has_correction = bool(params.get("correction", True))
        self.router_name = str(params.get("router_name", "router"))
        self.correction_name = str(params.get("correction_name", "correction"))
        self.expert_names = tuple(params.get("expert_names", ("e{index}.gate", "e{index}.up", "e{index}.down")))
        self.scoring = str(params.get("scoring", "sigmoid"))
        self.renormalise = bool(params.get("renormalise", False))
        self.identity_experts = int(params.get("identity_experts") or 0)
        shared = params.get("shared_intermediate_size")
        self.shared_intermediate_size = None if shared is None else int(shared)
        self.shared_names = tuple(params.get("shared_names", ("shared.gate", "shared.up", "shared.down")))
        self.router_outputs = self.num_experts + self.identity_experts
        self.activation = self._activation(params.get("activation", "silu"))
        self.shared_activation = self._activation(params.get("shared_activation", "silu"))
        self.weight_on_input = bool(params.get("weight_on_input", False))
        if self.weight_on_input and self.identity_experts:
            raise ValueError("identity experts take their weight on what they return: weight_on_input=False")
        if self.scoring not in ("sigmoid", "softmax"):
            raise ValueError(f"router scores {self.scoring!r}: 'sigmoid' or 'softmax'")
        if self.identity_experts < 0 or self.num_experts < 1:
            raise ValueError(f"{self.num_experts} experts and {self.identity_experts} identity experts")
        if not 1 <= self.top <= self.router_outputs:
            raise ValueError(f"top={self.top} of {self.router_outputs} experts")
        if self.group_count < 1 or self.router_outputs % self.group_count:
            raise ValueError(f"{self.router_outputs} experts do not form {self.group_count} equal groups")
        if not 1 <= self.group_keep <= self.group_count:
            raise ValueError(f"group_keep={self.group_keep} of {self.group_count} groups")
        if self.top > self.group_keep * (self.router_outputs // self.group_count):
            raise ValueError(f"top={self.top} experts cannot come from {self.group_keep} groups of "
                             f"{self.router_outputs // self.group_count}")
        self.router = self.correction = self.gate_up = self.down = self.shared_gate_up = self.shared_down = None

    @staticmethod
    def _activation(value):
        if value == "silu":
            return "silu"
        value = tuple(value)
        if len(value) != 4 or value[0] != "capped":
            raise ValueError(f"an expert's activation is 'silu' or ('capped', limit, slope, offset), not {value!r}")
        return ("capped", float(value[1]), float(value[2]), float(value[3]))

    def _expert(self, index: int) -> tuple[str, str, str]:
        return tuple(pattern.format(index=index) for pattern in self.expert_names)

    def expected_weights(self) -> dict[str, WeightInfo]:
        inter, hidden = self.intermediate_size, self.env.hidden_size
        # the router's matrix is used in 32-bit arithmetic: kept in float32 like a norm's vector
        names = {self.router_name: WeightInfo((self.router_outputs, hidden), "vector")}
        if self.has_correction:
            names[self.correction_name] = WeightInfo((self.router_outputs,), "vector")
        if self.shared_intermediate_size is not None:
            gate, up, down = self.shared_names
            names[gate] = WeightInfo((self.shared_intermediate_size, hidden))
            names[up] = WeightInfo((self.shared_intermediate_size, hidden))
            names[down] = WeightInfo((hidden, self.shared_intermediate_size))
        for index in range(self.num_experts):
            gate, up, down = self._expert(index)
            names[gate] = WeightInfo((inter, hidden))
            names[up] = WeightInfo((inter, hidden))
            names[down] = WeightInfo((hidden, inter))
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.router = tensors[self.router_name].contiguous()
        self.correction = tensors[self.correction_name].contiguous() if self.has_correction else None
        names = [self._expert(index) for index in range(self.num_experts)]
        self.gate_up = torch.stack([torch.cat([tensors[gate], tensors[up]], dim=0) for gate, up, _ in names]).contiguous()
        self.down = torch.stack([tensors[down] for _, _, down in names]).contiguous()
        if self.shared_intermediate_size is not None:
            gate, up, down = self.shared_names
            self.shared_gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()
            self.shared_down = tensors[down].contiguous()

    # From this many rows over all lists on, bfloat16 products whose sizes the library takes go to it.
    LIBRARY_MIN_ROWS = 256

    def _library_takes(self, x: torch.Tensor, rows: int) -> bool:
        return (x.dtype == torch.bfloat16 and rows >= self.LIBRARY_MIN_ROWS and hasattr(torch, "_grouped_mm")
                and x.shape[1] % 8 == 0 and self.intermediate_size % 8 == 0)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from ..kernels import grouped
        tokens, device = x.shape[0], x.device
        top, experts = self.top, self.num_experts
        ids = torch.empty((tokens, top), dtype=torch.int32, device=device)
        weights = torch.empty((tokens, top), dtype=torch.float32, device=device)
        grouped.route_experts(x, self.router, self.correction, ids, weights, top, self.group_count,
                              self.group_keep, self.group_top, scoring=self.scoring, renormalise=self.renormalise)
        # three words ahead of the offsets, so that offsets[1:] (where each list ends) begins at 16 bytes
        books = torch.empty(3 + experts + 1 + 2 * tokens * top, dtype=torch.int32, device=device)
        _, offsets, sorted_pair, position = torch.split(books, [3, experts + 1, tokens * top, tokens * top])
        grouped.expert_lists(ids, experts, offsets, sorted_pair, position)
        hidden = torch.empty((tokens * top, self.intermediate_size), dtype=x.dtype, device=device)
        if self._library_takes(x, tokens * top):
            # Many rows: the library's grouped product over the rows put side by side list by list (as the
            # engine's large plain products go to the library), the activation as a kernel of its own.
            gathered = torch.empty((tokens * top, x.shape[1]), dtype=x.dtype, device=device)
            grouped.gather_rows(x, sorted_pair, top, gathered)
            gate_up = torch._grouped_mm(gathered, self.gate_up.transpose(1, 2), offs=offsets[1:])
            kernels.count_launch()
            scale = (weights, sorted_pair) if self.weight_on_input else (None, None)
            if self.activation == "silu" and not self.weight_on_input:
                kernels.silu_mul(gate_up, hidden)
            elif self.activation == "silu":     # silu is the capped form without a cap: slope 1, nothing added
                grouped.capped_swish_mul(gate_up, hidden, None, 1.0, 0.0, *scale)
            else:
                grouped.capped_swish_mul(gate_up, hidden, *self.activation[1:], *scale)
            rows = torch._grouped_mm(hidden, self.down.transpose(1, 2), offs=offsets[1:])
            kernels.count_launch()
        else:
            rows = torch.empty((tokens * top, self.env.hidden_size), dtype=x.dtype, device=device)
            grouped.expert_gemm(x, self.gate_up, hidden, offsets, sorted_pair, top, gated=self.activation,
                                row_scale=weights if self.weight_on_input else None)
            grouped.expert_gemm(hidden, self.down, rows, offsets, None)
        shared = None
        if self.shared_gate_up is not None:
            inner = torch.empty((tokens, self.shared_intermediate_size), dtype=x.dtype, device=device)
            if self.shared_activation == "silu":
                kernels.gated_silu_gemm(x, self.shared_gate_up, inner)
            else:
                both = torch.empty((tokens, 2 * self.shared_intermediate_size), dtype=x.dtype, device=device)
                kernels.gemm(x, self.shared_gate_up, both)
                grouped.capped_swish_mul(both, inner, *self.shared_activation[1:])
            shared = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=device)
            kernels.gemm(inner, self.shared_down, shared)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=device)
        # An identity expert's pairs have numbers past the lists' (no row: `position` is negative); the last
        # kernel adds the token's own input for them, and the shared expert's row.
        identity = (ids, x, experts) if self.identity_experts else None
        grouped.combine_experts(rows, position, None if self.weight_on_input else weights, out, identity=identity,
                                extra=shared, top=top)
        return out
