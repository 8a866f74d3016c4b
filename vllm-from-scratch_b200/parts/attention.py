"""Causal attention over a paged cache, with grouped key/value heads, optional
per-head RMSNorm of queries and keys, and an optional window.

Computation (minivllm/models/qwen3.py:103-124): one product for queries, keys and
values (rows ``[Q; K; V]`` of one matrix, minivllm/layers/linear.py:209-214) ->
per-head norm over ``head_dim`` with one weight vector for all heads -> position
encoding on queries and keys -> keys and values stored at the new tokens' slots ->
softmax(q k^T * scale + causal mask) v over everything the request has cached
(minivllm/attention/backends/torch_sdpa.py:450-489) -> output product.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import (MIXERS, CacheView, HalfNormedRows, KVPagesNeed, Mixer, Norm, PartEnv, PositionEncoding,
                   StepContext, WeightInfo)


@MIXERS.register("paged_attention")
class PagedAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale`` (default
    ``head_dim ** -0.5``), ``window`` (None = all keys), ``qk_norm_eps`` (None =
    no per-head norm)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        window = params.get("window")
        self.window = None if window is None else int(window)
        eps = params.get("qk_norm_eps")
        self.qk_norm_eps = None if eps is None else float(eps)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads={self.num_heads} is not a multiple of num_kv_heads={self.num_kv_heads}")
        if self.head_dim % 2 or self.head_dim > 512:
            raise ValueError(f"head_dim={self.head_dim}: the attention kernels take even sizes up to 512")
        if position.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim={position.rotary_dim} exceeds head_dim={self.head_dim}")
        if getattr(position, "interleaved", False):
            raise ValueError("this mixer's kernels turn halves of a head, not neighbours: interleaved=False")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        self.qkv: torch.Tensor | None = None
        self.out_proj: torch.Tensor | None = None
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None

    # ------------------------------------------------------------------ weights
    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, d = self.env.hidden_size, self.head_dim
        names = {
            "q_proj.weight": WeightInfo((self.num_heads * d, hidden)),
            "k_proj.weight": WeightInfo((self.num_kv_heads * d, hidden)),
            "v_proj.weight": WeightInfo((self.num_kv_heads * d, hidden)),
            "o_proj.weight": WeightInfo((hidden, self.num_heads * d)),
        }
        if self.qk_norm_eps is not None:
            names["q_norm.weight"] = WeightInfo((d,), "vector")
            names["k_norm.weight"] = WeightInfo((d,), "vector")
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                              tensors["v_proj.weight"]], dim=0).contiguous()
        self.out_proj = tensors["o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors["q_norm.weight"], tensors["k_norm.weight"]

    # -------------------------------------------------------------------- cache
    def cache_need(self) -> KVPagesNeed:
        return KVPagesNeed(self.num_kv_heads, self.head_dim, self.window)

    # ------------------------------------------------------------------ forward
    def splits_norms(self, tokens: int) -> bool:
        return (kernels.split_norm_ok(tokens, self.qkv, fold=False)
                and kernels.split_norm_ok(tokens, self.out_proj, fold=True))

    def forward(self, x: torch.Tensor | HalfNormedRows, ctx: StepContext, cache: CacheView,
                fold: tuple[torch.Tensor, Norm] | None = None) -> torch.Tensor | HalfNormedRows:
        if cache.kind != "pages":
            raise ValueError("paged attention needs a cache of pages")
        group = ctx.groups[cache.group]
        scale = (x.squares, x.eps) if isinstance(x, HalfNormedRows) else None
        x = x.rows if isinstance(x, HalfNormedRows) else x
        tokens = x.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = torch.empty((tokens, (nq + 2 * nkv) * d), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.qkv, qkv, scale=scale)
        store = cache.writable
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        rope = (self.q_norm, self.k_norm, self.position.inverse_frequencies(), self.position.rotary_dim, eps)
        attended = torch.empty((tokens, nq * d), dtype=x.dtype, device=x.device)
        # Requests that bring one token (all of a decode step, the first ctx.num_decode of a
        # mixed one): norms, rotation, the store of the new key and value and the attention
        # in one kernel, where there is one for the shape.
        single = tokens if ctx.max_query_len == 1 and tokens == ctx.num_requests else ctx.num_decode
        fused = 0
        if store and single > 0 and kernels.fused_decode_attention(
                qkv[:single], ctx.positions[:single], group.slot_mapping[:single], *rope, cache.keys, cache.values,
                attended[:single], ctx.seq_lens[:single], group.block_table[:single], nq, nkv, d, group.page_size,
                self.scale, self.window, ctx.max_seq_len):
            fused = single
        if fused < tokens:
            q = torch.empty((tokens, nq * d), dtype=x.dtype, device=x.device)
            kernels.head_norm_rope_cache(
                qkv[fused:], ctx.positions[fused:], group.slot_mapping[fused:], *rope, q[fused:],
                cache.keys if store else None, cache.values if store else None, nq, nkv, d, group.page_size)
            kernels.paged_attention(
                q, cache.keys, cache.values, attended, ctx.query_start, ctx.seq_lens, group.block_table,
                nq, nkv, d, group.page_size, self.scale, self.window, ctx.max_query_len, ctx.max_seq_len,
                ctx.num_decode, decode_done=fused > 0)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        if fold is None:
            kernels.gemm(attended, self.out_proj, out)
            return out
        residual, norm = fold
        weight, eps = norm.split()
        squares = torch.empty((tokens, self.env.hidden_size // 8), dtype=torch.float32, device=x.device)
        kernels.gemm(attended, self.out_proj, out, fold=(residual, weight, squares))
        return HalfNormedRows(out, squares, eps)


def power_of_two_slopes(num_heads: int, span: float = 8.0) -> list[float]:
    """``2 ** (-span * (h + 1) / num_heads)`` for head h: the slopes of a linear distance bias."""
    return [2.0 ** (-span * (head + 1) / num_heads) for head in range(num_heads)]


@MIXERS.register("biased_attention")
class BiasedAttention(Mixer):
    """Causal softmax attention over a paged cache in which positions enter as a bias on the
    scores, not as a rotation: ``score(i, j) = q_i . k_j * scale - slope_h * (i - j)``.  Grouped
    key/value heads; keys and values may have sizes of their own; optional per-head RMSNorm of
    queries and keys (one plain weight vector for all heads); optional query temperature ``1 + coef
    * ln(floor((p + 1) / every) + 1)`` at position p.  Scores, softmax weights and the weighted sum
    are float32 in both run modes.

    params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim`` (default ``head_dim``),
    ``scale``, ``slopes`` (one per head, or None for no bias), ``window`` (None = all keys),
    ``qk_norm_eps`` (None = no head norm), ``qk_norm_weights`` (default True; False: queries and keys are
    divided by their root mean square and nothing else, the checkpoint has no vectors for it),
    ``q_temperature`` (``(coef, every)`` or None), ``cache_window`` (positions the cache keeps, where
    another layer reads it over a longer window than this one's; default: the window),
    ``weight_names`` (q, k, v, o matrices, q and k norm vectors)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        if position.rotary_dim:
            raise ValueError("biased attention takes no rotation: give it position encoding 'none'")
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        window = params.get("window")
        self.window = None if window is None else int(window)
        eps = params.get("qk_norm_eps")
        self.qk_norm_eps = None if eps is None else float(eps)
        self.qk_norm_weights = bool(params.get("qk_norm_weights", True))
        self.cache_window = params.get("cache_window", self.window)
        temperature = params.get("q_temperature")
        self.q_temperature = None if temperature is None else (float(temperature[0]), int(temperature[1]))
        slopes = params.get("slopes")
        self.slopes_host = None if slopes is None else [float(s) for s in slopes]
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads={self.num_heads} is not a multiple of num_kv_heads={self.num_kv_heads}")
        if self.head_dim > 512 or self.value_dim > 512:
            raise ValueError(f"head_dim={self.head_dim}, value_dim={self.value_dim}: sizes up to 512 are built")
        if self.slopes_host is not None and len(self.slopes_host) != self.num_heads:
            raise ValueError(f"{len(self.slopes_host)} slopes for {self.num_heads} heads")
        if self.q_temperature is not None and self.q_temperature[1] <= 0:
            raise ValueError(f"q_temperature every={self.q_temperature[1]} must be positive")
        self.names = tuple(params.get("weight_names", ("q_proj.weight", "k_proj.weight", "v_proj.weight",
                                                       "o_proj.weight", "q_norm.weight", "k_norm.weight")))
        self.slopes = (None if self.slopes_host is None
                       else torch.tensor(self.slopes_host, dtype=torch.float64).to(torch.float32).to(env.device))
        self.qkv = self.out_proj = self.q_norm = self.k_norm = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, d, dv = self.env.hidden_size, self.head_dim, self.value_dim
        q, k, v, o, qn, kn = self.names
        names = {q: WeightInfo((self.num_heads * d, hidden)), k: WeightInfo((self.num_kv_heads * d, hidden)),
                 v: WeightInfo((self.num_kv_heads * dv, hidden)), o: WeightInfo((hidden, self.num_heads * dv))}
        if self.qk_norm_eps is not None and self.qk_norm_weights:
            names[qn] = WeightInfo((d,), "vector")
            names[kn] = WeightInfo((d,), "vector")
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        q, k, v, o, qn, kn = self.names
        self.qkv = torch.cat([tensors[q], tensors[k], tensors[v]], dim=0).contiguous()
        self.out_proj = tensors[o].contiguous()
        if self.qk_norm_eps is not None and self.qk_norm_weights:
            self.q_norm, self.k_norm = tensors[qn], tensors[kn]

    def cache_need(self) -> KVPagesNeed:
        return KVPagesNeed(self.num_kv_heads, self.head_dim, self.cache_window, self.value_dim)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if cache.kind != "pages":
            raise ValueError("biased attention needs a cache of pages")
        group = ctx.groups[cache.group]
        tokens = x.shape[0]
        nq, nkv, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        qkv = torch.empty((tokens, self.qkv.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.qkv, qkv)
        q = torch.empty((tokens, nq * d), dtype=x.dtype, device=x.device)
        store = cache.writable
        kernels.head_norm_scale_cache(
            qkv, ctx.positions, group.slot_mapping, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0,
            self.q_temperature, q, cache.keys if store else None, cache.values if store else None, nq, nkv, d, dv,
            group.page_size, unit_norm=self.qk_norm_eps is not None and not self.qk_norm_weights)
        attended = torch.empty((tokens, nq * dv), dtype=x.dtype, device=x.device)
        kernels.biased_paged_attention(
            q, cache.keys, cache.values, attended, ctx.query_start, ctx.seq_lens, group.block_table, self.slopes,
            nq, nkv, d, dv, group.page_size, self.scale, self.window, ctx.max_query_len, ctx.max_seq_len,
            ctx.num_decode)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(attended, self.out_proj, out)
        return out


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """Causal attention over a paged cache in which every head has two softmax maps over the same values, the
    second subtracted from the first: with ``a_m = softmax_j(cap(q_m . k_mj * scale)) v_j`` for the maps m = 1, 2
    (queries and keys of ``head_dim`` numbers each, laid out ``[map 1, map 2]`` head by head in the projections),
    ``o = a1 - lam * a2``, then ``o * rsqrt(mean(o^2) + norm_eps) * (1 - diff)`` over the head's ``value_dim`` values,
    then the output product over the heads side by side.  ``lam = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) +
    diff`` is one number for the layer, formed once from four vectors of ``head_dim`` numbers.

    Scores are capped (``cap(s) = softcap * tanh(s / softcap)``; None: not capped); a query at position i sees the
    keys ``j <= i`` with ``i - j < window`` and, whatever the window, the first ``keep_first`` positions of the
    sequence, all at their true positions.  The position encoding (rotary family) rotates the first ``rotary_dim``
    numbers of every map of every query and key head; the projections of queries, keys and values have biases
    (``bias``, default True).  Grouped heads: query head h reads key/value head ``h // (num_heads //
    num_kv_heads)``.  Scores, weights, the weighted sums, the difference and its norm are float32 in both run
    modes.

    params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``softcap``, ``window``,
    ``keep_first`` (default 0), ``diff``, ``norm_eps``, ``bias``, ``weight_names`` (q, k, v, o matrices and the
    vectors lq1, lk1, lq2, lk2; a bias is its matrix's name with ``bias_suffix``, default ``.b``, behind it)."""

    graph_safe = True
    MAPS = 2

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        softcap = params.get("softcap")
        self.softcap = None if softcap is None else float(softcap)
        window = params.get("window")
        self.window = None if window is None else int(window)
        self.keep_first = int(params.get("keep_first") or 0) if self.window is not None else 0
        self.diff = float(params["diff"])
        self.norm_eps = float(params["norm_eps"])
        self.has_bias = bool(params.get("bias", True))
        self.bias_suffix = str(params.get("bias_suffix", ".b"))
        self.names = tuple(params.get("weight_names", ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")))
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads={self.num_heads} is not a multiple of num_kv_heads={self.num_kv_heads}")
        if self.MAPS * self.head_dim > 1024 or self.value_dim > 512:
            raise ValueError(f"head_dim={self.head_dim}, value_dim={self.value_dim}: maps up to 512 and values up to "
                             f"512 are built")
        if position.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim={position.rotary_dim} exceeds head_dim={self.head_dim}")
        if getattr(position, "interleaved", False):
            raise ValueError("this mixer's kernels turn halves of a head, not neighbours: interleaved=False")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        if self.softcap is not None and self.softcap <= 0:
            raise ValueError(f"softcap must be positive, got {self.softcap}")
        self.qkv = self.out_proj = self.bias = None
        self.lam = 0.0

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, d, dv, maps = self.env.hidden_size, self.head_dim, self.value_dim, self.MAPS
        q, k, v, o = self.names[:4]
        rows = {q: self.num_heads * maps * d, k: self.num_kv_heads * maps * d, v: self.num_kv_heads * dv}
        names = {name: WeightInfo((count, hidden)) for name, count in rows.items()}
        names[o] = WeightInfo((hidden, self.num_heads * dv))
        if self.has_bias:
            for name, count in rows.items():
                names[name + self.bias_suffix] = WeightInfo((count,), "vector")
        for name in self.names[4:]:
            names[name] = WeightInfo((d,), "vector")
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        q, k, v, o, lq1, lk1, lq2, lk2 = self.names
        self.qkv = torch.cat([tensors[q], tensors[k], tensors[v]], dim=0).contiguous()
        self.out_proj = tensors[o].contiguous()
        if self.has_bias:
            self.bias = torch.cat([tensors[name + self.bias_suffix] for name in (q, k, v)]).contiguous()
        first = torch.exp((tensors[lq1] * tensors[lk1]).sum())      # float32 vectors: one number, formed once
        second = torch.exp((tensors[lq2] * tensors[lk2]).sum())
        self.lam = float((first - second + self.diff).item())

    def cache_need(self) -> KVPagesNeed:
        # a position's keys of both maps lie side by side in one row of its key/value head
        return KVPagesNeed(self.num_kv_heads, self.MAPS * self.head_dim, self.window, self.value_dim,
                           keep_first=self.keep_first)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        from ..kernels import differential
        if cache.kind != "pages":
            raise ValueError("differential attention needs a cache of pages")
        group = ctx.groups[cache.group]
        tokens = x.shape[0]
        nq, nkv, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        qkv = torch.empty((tokens, self.qkv.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.qkv, qkv)
        q = torch.empty((tokens, nq * self.MAPS * d), dtype=x.dtype, device=x.device)
        store = cache.writable
        differential.bias_rope_cache(
            qkv, self.bias, ctx.positions, group.slot_mapping, self.position.inverse_frequencies(),
            self.position.rotary_dim, q, cache.keys if store else None, cache.values if store else None, nq, nkv, d, dv,
            group.page_size)
        attended = torch.empty((tokens, nq * dv), dtype=x.dtype, device=x.device)
        differential.diff_paged_attention(
            q, cache.keys, cache.values, attended, ctx.query_start, ctx.seq_lens, group.block_table, nq, nkv, d, dv,
            group.page_size, self.scale, self.softcap, self.window, self.keep_first, self.lam, self.norm_eps,
            1.0 - self.diff, ctx.max_query_len, ctx.max_seq_len, ctx.num_decode)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(attended, self.out_proj, out)
        return out
