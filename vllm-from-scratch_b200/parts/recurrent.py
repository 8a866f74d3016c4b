"""Mixers that carry a matrix of state per head from token to token instead of a cache of keys.

``decayed_linear_attention``: ``S <- decay_h S + k v^T``, ``o = S^T q`` with q, k, v = silu of their
projections and a constant decay per head; the heads' outputs, side by side, pass one RMSNorm, a
sigmoid gate and the output product.

``selective_scan``: one input product laid out ``[z | x | B | C | dt]``; x, B and C pass a short causal
convolution per channel and silu; ``dt = softplus(dt + bias)``; per head ``S <- exp(-exp(A_log) dt) S + dt
B x^T``, ``y = S^T C + D x`` (B and C shared by the heads of a group); ``y * silu(z)`` is normalised in
equal parts, each by its own root mean square, weighted and projected.

``gated_linear_attention``: ``S <- diag(a) S + k v^T``, ``o = S^T q`` with ``q = W_q h * head_dim ** -0.5``, k and v
as projected, and a decay per head and key channel ``a = sigmoid(z) ** (1 / tau)``, ``z = W_a2 (W_a1 h) + b`` through
two small matrices; every head's output passes an RMSNorm of its own (one weight vector of ``value_dim`` numbers for
all heads), the heads side by side are multiplied by ``silu(W_g h)`` and projected.

All keep their state as float32 ``[slots, heads, N, value_dim]`` in the cache's state slots and
compute decays, step sizes, gates and norms in float32 in both run modes; a prompt may arrive in any
portions (the kernels read the state of a request's slot before its first token of the step and
leave it advanced).
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import MIXERS, CacheView, Mixer, PartEnv, PositionEncoding, StateNeed, StepContext, WeightInfo


@MIXERS.register("decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """params: ``num_heads``, ``head_dim`` (queries and keys), ``value_dim``, ``decay`` (one constant per
    head), ``norm_eps``, ``weight_names`` (q, k, v, gate, output matrices and the norm vector; default
    ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params["value_dim"])
        self.norm_eps = float(params["norm_eps"])
        decay = [float(value) for value in params["decay"]]
        if len(decay) != self.num_heads:
            raise ValueError(f"{len(decay)} decay constants for {self.num_heads} heads")
        if self.head_dim > 256:
            raise ValueError(f"head_dim={self.head_dim}: the recurrence kernel holds up to 256 rows of state a head")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(env.device)
        self.names = tuple(params.get("weight_names", ("q", "k", "v", "g", "o", "norm")))
        self.qkvg = self.out_proj = self.norm = None

    @property
    def inner(self) -> int:
        return self.num_heads * self.value_dim

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, keys = self.env.hidden_size, self.num_heads * self.head_dim
        q, k, v, g, o, norm = self.names
        return {q: WeightInfo((keys, hidden)), k: WeightInfo((keys, hidden)), v: WeightInfo((self.inner, hidden)),
                g: WeightInfo((self.inner, hidden)), o: WeightInfo((hidden, self.inner)),
                norm: WeightInfo((self.inner,), "vector")}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        q, k, v, g, o, norm = self.names
        # One product for all four projections; the gate first, so that its columns start a row.
        self.qkvg = torch.cat([tensors[g], tensors[q], tensors[k], tensors[v]], dim=0).contiguous()
        self.out_proj = tensors[o].contiguous()
        self.norm = tensors[norm]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.num_heads, self.head_dim, self.value_dim), torch.float32, name="state")

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        state = cache.states.get("state") if cache.states else cache.state
        if state is None:
            raise ValueError("decayed linear attention needs its state slots")
        tokens = x.shape[0]
        keys = self.num_heads * self.head_dim
        proj = torch.empty((tokens, self.qkvg.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.qkvg, proj)
        y = torch.empty((tokens, self.inner), dtype=torch.float32, device=x.device)
        kernels.decayed_linear_attention(proj, (self.inner, self.inner + keys, self.inner + 2 * keys), self.decay,
                                         ctx.query_start, ctx.state_slots, state, y, self.num_heads, self.head_dim,
                                         self.value_dim, ctx.max_query_len)
        gated = torch.empty((tokens, self.inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(y, proj, self.norm, gated, 1, False, self.norm_eps)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(gated, self.out_proj, out)
        return out


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """params: ``num_heads``, ``head_dim`` (queries and keys), ``value_dim``, ``tau``, ``norm_eps``, ``out_scale`` (a
    factor on the gated rows ahead of the output product; default 1), ``weight_names`` (q, k, v, gate, output
    matrices, the norm vector, the decay's two matrices and its bias; default ``q``, ``k``, ``v``, ``g``, ``o``,
    ``norm``, ``a1``, ``a2``, ``a2.b``).  The rank of the decay's matrices is the checkpoint's."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params["value_dim"])
        self.tau = float(params["tau"])
        self.norm_eps = float(params["norm_eps"])
        self.out_scale = float(params.get("out_scale", 1.0))
        if self.tau <= 0:
            raise ValueError(f"tau={self.tau} must be positive")
        if self.head_dim > 256:
            raise ValueError(f"head_dim={self.head_dim}: the recurrence kernel holds up to 256 rows of state a head")
        self.names = tuple(params.get("weight_names", ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b")))
        self.qkvg = self.down = self.up = self.up_bias = self.out_proj = self.norm = None

    @property
    def inner(self) -> int:
        return self.num_heads * self.value_dim

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, keys = self.env.hidden_size, self.num_heads * self.head_dim
        q, k, v, g, o, norm, a1, a2, a2_bias = self.names
        return {q: WeightInfo((keys, hidden)), k: WeightInfo((keys, hidden)), v: WeightInfo((self.inner, hidden)),
                g: WeightInfo((self.inner, hidden)), o: WeightInfo((hidden, self.inner)),
                norm: WeightInfo((self.value_dim,), "vector"),
                a1: WeightInfo((None, hidden)), a2: WeightInfo((keys, None)), a2_bias: WeightInfo((keys,), "vector")}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        q, k, v, g, o, norm, a1, a2, a2_bias = self.names
        if tensors[a1].shape[0] != tensors[a2].shape[1]:
            raise ValueError(f"the decay's matrices {tuple(tensors[a1].shape)} and {tuple(tensors[a2].shape)} do not "
                             f"share a rank")
        # One product for the gate, q, k and v; the gate first, so that its columns start a row.
        self.qkvg = torch.cat([tensors[g], tensors[q], tensors[k], tensors[v]], dim=0).contiguous()
        self.down = tensors[a1].contiguous()
        self.up = tensors[a2].contiguous()
        self.up_bias = tensors[a2_bias].contiguous()
        self.out_proj = tensors[o].contiguous()
        self.norm = tensors[norm].repeat(self.num_heads).contiguous()       # every head's part of a row has the vector
        self._scaled_norms = {1.0: self.norm}

    def cache_need(self) -> StateNeed:
        return StateNeed((self.num_heads, self.head_dim, self.value_dim), torch.float32, name="state")

    def inner_width(self) -> int:
        return self.inner

    def forward_inner(self, x: torch.Tensor, ctx: StepContext, cache: CacheView, factor: float = 1.0,
                      out: torch.Tensor | None = None) -> torch.Tensor:
        """The normalised, gated heads side by side, times ``factor``: what the output product multiplies.  ``out``:
        where to write them, ``[T, heads * value_dim]``, which may be columns of wider rows."""
        state = cache.states.get("state") if cache.states else cache.state
        if state is None:
            raise ValueError("gated linear attention needs its state slots")
        tokens = x.shape[0]
        keys = self.num_heads * self.head_dim
        proj = torch.empty((tokens, self.qkvg.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.qkvg, proj)
        low = torch.empty((tokens, self.down.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.down, low)
        logits = torch.empty((tokens, keys), dtype=x.dtype, device=x.device)
        kernels.gemm(low, self.up, logits)
        y = torch.empty((tokens, self.inner), dtype=torch.float32, device=x.device)
        kernels.gated_linear_attention(proj, (self.inner, self.inner + keys, self.inner + 2 * keys), logits, 0,
                                       self.up_bias, self.tau, self.head_dim ** -0.5, ctx.query_start,
                                       ctx.state_slots, state, y, self.num_heads, self.head_dim, self.value_dim,
                                       ctx.max_query_len)
        gated = out if out is not None else torch.empty((tokens, self.inner), dtype=x.dtype, device=x.device)
        factor = factor * self.out_scale
        if factor not in self._scaled_norms:        # the factor rides on the norm's weights (float32, formed once)
            self._scaled_norms[factor] = (self.norm * factor).contiguous()
        kernels.gated_group_norm(y, proj, self._scaled_norms[factor], gated, self.num_heads, False, self.norm_eps,
                                 silu_behind=True)
        return gated

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        inner = self.forward_inner(x, ctx, cache)
        out = torch.empty((x.shape[0], self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(inner, self.out_proj, out)
        return out


@MIXERS.register("selective_scan")
class SelectiveScan(Mixer):
    """params: ``num_heads``, ``value_dim`` (per head; inner = heads * value_dim), ``state_dim`` (N),
    ``groups`` (of heads that share B and C), ``conv_taps``, ``norm_groups``, ``norm_eps``,
    ``weight_names`` (input matrix, conv weight and bias, dt bias, A_log, D, norm vector, output matrix;
    default ``in``, ``conv``, ``conv.b``, ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.value_dim = int(params["value_dim"])
        self.state_dim = int(params["state_dim"])
        self.groups = int(params["groups"])
        self.taps = int(params["conv_taps"])
        self.norm_groups = int(params["norm_groups"])
        self.norm_eps = float(params["norm_eps"])
        self.inner = self.num_heads * self.value_dim
        self.channels = self.inner + 2 * self.groups * self.state_dim
        if self.num_heads % self.groups:
            raise ValueError(f"num_heads={self.num_heads} is not a multiple of groups={self.groups}")
        if self.inner % self.norm_groups:
            raise ValueError(f"inner width {self.inner} does not divide into {self.norm_groups} norm groups")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"conv_taps={self.taps}: 1 to 16 are built")
        if self.state_dim > 256:
            raise ValueError(f"state_dim={self.state_dim}: the recurrence kernel holds up to 256 rows of state a head")
        self.names = tuple(params.get("weight_names", ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")))
        self.in_proj = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm = self.out_proj = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, heads = self.env.hidden_size, self.num_heads
        w_in, conv, conv_b, dt_bias, a_log, skip, norm, out = self.names
        return {w_in: WeightInfo((self.inner + self.channels + heads, hidden)),
                conv: WeightInfo((self.channels, self.taps), "vector"), conv_b: WeightInfo((self.channels,), "vector"),
                dt_bias: WeightInfo((heads,), "vector"), a_log: WeightInfo((heads,), "vector"),
                skip: WeightInfo((heads,), "vector"), norm: WeightInfo((self.inner,), "vector"),
                out: WeightInfo((hidden, self.inner))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w_in, conv, conv_b, dt_bias, a_log, skip, norm, out = self.names
        self.in_proj = tensors[w_in].contiguous()
        # tap by tap, [taps, channels]: the kernel's warps read a tap's weights side by side
        self.conv, self.conv_bias = tensors[conv].t().contiguous(), tensors[conv_b]
        self.dt_bias, self.a_log, self.skip = tensors[dt_bias], tensors[a_log], tensors[skip]
        self.norm = tensors[norm]
        self.out_proj = tensors[out].contiguous()

    def cache_need(self) -> tuple[StateNeed, StateNeed]:
        return (StateNeed((self.num_heads, self.state_dim, self.value_dim), torch.float32, name="state"),
                StateNeed((self.taps - 1, self.channels), torch.float32, name="conv"))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if "state" not in cache.states or "conv" not in cache.states:
            raise ValueError("the selective scan needs its two state tensors (recurrence and convolution)")
        tokens = x.shape[0]
        proj = torch.empty((tokens, self.in_proj.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.in_proj, proj)
        xbc = torch.empty((tokens, self.channels), dtype=torch.float32, device=x.device)
        kernels.causal_conv_silu(proj, self.inner, self.conv, self.conv_bias, cache.states["conv"],
                                 ctx.token_request, ctx.query_start, ctx.state_slots, xbc)
        y = torch.empty((tokens, self.inner), dtype=torch.float32, device=x.device)
        kernels.selective_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.skip,
                               ctx.query_start, ctx.state_slots, cache.states["state"], y, self.num_heads,
                               self.groups, self.state_dim, self.value_dim, ctx.max_query_len)
        gated = torch.empty((tokens, self.inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(y, proj, self.norm, gated, self.norm_groups, True, self.norm_eps)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(gated, self.out_proj, out)
        return out
