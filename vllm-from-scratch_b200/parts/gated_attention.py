"""Causal softmax attention over a paged cache whose heads' outputs pass a gate of their own, with the forms of
projection, norm, rotation and softmax as parameters:

* ``bias``: the projections of queries, keys and values have bias vectors (added in float32);
* ``qk_norm``: RMSNorm of queries and keys, ``"head"`` (over each head, one plain weight vector of ``head_dim`` numbers
  for all heads), ``"whole"`` (over all heads of the projection at once, plain weight vectors of its whole size) or
  None; before any rotation;
* the position encoding (rotary family) turns the first ``rotary_dim`` numbers of every query and key head, as
  neighbours or as halves (the encoding's ``interleaved``);
* ``window``: position i sees the keys j with ``0 <= i - j < window`` (None: every earlier key);
* ``unit_sink``: one is added to the softmax denominator, ``p_j = exp(s_j) / (1 + sum exp(s))``: a sink whose score is
  0 and which has no value;
* ``output_gate``: head h's output is multiplied by ``sigmoid(W_g x)_h``, one number per head from the mixer's own
  input, ahead of the output product;
* ``own_kv=False``: the layer has no projections of keys and values and reads the pages another layer wrote (the
  schedule entry names the owner in ``cache_from``), with queries, window and gate of its own.

Scores, softmax weights, the weighted sum of the values, norms, angles and gates are float32 in both run modes.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import MIXERS, CacheView, KVPagesNeed, Mixer, PartEnv, PositionEncoding, StepContext, WeightInfo


@MIXERS.register("gated_softmax_attention")
class GatedSoftmaxAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim`` (default ``head_dim``), ``scale``,
    ``window`` (None = all keys), ``cache_window`` (positions the cache keeps where a reader's window is longer than
    the owner's; default: the window), ``bias`` (default False), ``bias_suffix`` (default ``.b``), ``qk_norm`` (None,
    ``"head"`` or ``"whole"``), ``qk_norm_eps``, ``unit_sink`` (default False), ``output_gate`` (default True),
    ``own_kv`` (default True), ``out_scale`` (a factor on the heads' outputs, applied with the gate; default 1),
    ``weight_names`` (q, k, v, o matrices, q and k norm vectors, gate matrix; default ``q``, ``k``, ``v``, ``o``,
    ``q.norm``, ``k.norm``, ``g``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        window = params.get("window")
        self.window = None if window is None else int(window)
        self.cache_window = params.get("cache_window", self.window)
        self.has_bias = bool(params.get("bias", False))
        self.bias_suffix = str(params.get("bias_suffix", ".b"))
        self.qk_norm = params.get("qk_norm")
        self.qk_norm_eps = float(params.get("qk_norm_eps", 0.0))
        self.unit_sink = bool(params.get("unit_sink", False))
        self.output_gate = bool(params.get("output_gate", True))
        self.own_kv = bool(params.get("own_kv", True))
        self.out_scale = float(params.get("out_scale", 1.0))
        self.names = tuple(params.get("weight_names", ("q", "k", "v", "o", "q.norm", "k.norm", "g")))
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads={self.num_heads} is not a multiple of num_kv_heads={self.num_kv_heads}")
        if self.head_dim > 512 or self.value_dim > 512:
            raise ValueError(f"head_dim={self.head_dim}, value_dim={self.value_dim}: sizes up to 512 are built")
        if self.qk_norm not in (None, "head", "whole"):
            raise ValueError(f"qk_norm={self.qk_norm!r}: None, 'head' or 'whole'")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        if position.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim={position.rotary_dim} exceeds head_dim={self.head_dim}")
        self.proj = self.out_proj = self.bias = self.q_norm = self.k_norm = self.sinks = None

    # ------------------------------------------------------------------ weights
    def _rows(self) -> dict[str, int]:
        q, k, v = self.names[:3]
        rows = {q: self.num_heads * self.head_dim}
        if self.own_kv:
            rows[k] = self.num_kv_heads * self.head_dim
            rows[v] = self.num_kv_heads * self.value_dim
        return rows

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden = self.env.hidden_size
        q, k, v, o, qn, kn, g = self.names
        names = {name: WeightInfo((count, hidden)) for name, count in self._rows().items()}
        names[o] = WeightInfo((hidden, self.num_heads * self.value_dim))
        if self.has_bias:
            for name, count in self._rows().items():
                names[name + self.bias_suffix] = WeightInfo((count,), "vector")
        if self.qk_norm is not None:
            whole = self.qk_norm == "whole"
            names[qn] = WeightInfo((self.num_heads * self.head_dim if whole else self.head_dim,), "vector")
            if self.own_kv:
                names[kn] = WeightInfo((self.num_kv_heads * self.head_dim if whole else self.head_dim,), "vector")
        if self.output_gate:
            names[g] = WeightInfo((self.num_heads, hidden))
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        q, k, v, o, qn, kn, g = self.names
        rows = list(self._rows())
        # One product for queries, keys, values and the gates; the gates last, behind whole heads.
        self.proj = torch.cat([tensors[name] for name in rows] + ([tensors[g]] if self.output_gate else []),
                              dim=0).contiguous()
        self.out_proj = tensors[o].contiguous()
        if self.has_bias:
            self.bias = torch.cat([tensors[name + self.bias_suffix] for name in rows]).contiguous()
        if self.qk_norm is not None:
            self.q_norm = tensors[qn].contiguous()
            self.k_norm = tensors[kn].contiguous() if self.own_kv else None
        if self.unit_sink:
            self.sinks = torch.zeros(self.num_heads, dtype=torch.float32, device=self.out_proj.device)

    # -------------------------------------------------------------------- cache
    def cache_need(self) -> KVPagesNeed:
        # A layer that reads another's pages still says what it reads; the model gives it the owner's.
        return KVPagesNeed(self.num_kv_heads, self.head_dim, self.cache_window, self.value_dim)

    # ------------------------------------------------------------------ forward
    def inner_width(self) -> int:
        return self.num_heads * self.value_dim

    def forward_inner(self, x: torch.Tensor, ctx: StepContext, cache: CacheView, factor: float = 1.0,
                      out: torch.Tensor | None = None) -> torch.Tensor:
        """The heads' gated outputs side by side, times ``factor``: what the output product multiplies.  ``out``: where
        to write them, ``[T, heads * value_dim]``, which may be columns of wider rows."""
        if cache.kind != "pages":
            raise ValueError("attention needs a cache of pages")
        if cache.writable != self.own_kv:
            raise ValueError("a layer writes the pages it owns and only reads another layer's: "
                             f"own_kv={self.own_kv}, the cache is {'its own' if cache.writable else 'lent'}")
        group = ctx.groups[cache.group]
        tokens = x.shape[0]
        nq, nkv, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        projected = torch.empty((tokens, self.proj.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.proj, projected)
        q = torch.empty((tokens, nq * d), dtype=x.dtype, device=x.device)
        kernels.qk_prepare_cache(
            projected, self.bias, ctx.positions, group.slot_mapping, self.q_norm, self.k_norm, self.qk_norm,
            self.qk_norm_eps, self.position.inverse_frequencies(), self.position.rotary_dim,
            bool(getattr(self.position, "interleaved", False)), q, cache.keys if self.own_kv else None,
            cache.values if self.own_kv else None, nq, nkv if self.own_kv else 0, d, dv, group.page_size)
        attended = out if out is not None else torch.empty((tokens, nq * dv), dtype=x.dtype, device=x.device)
        factor = factor * self.out_scale
        # the gate (and the factor with it) is applied where the attention kernel writes a head's output
        gate = {"gate": projected, "gate_column": projected.shape[1] - nq, "gate_factor": factor} if self.output_gate else {}
        kernels.biased_paged_attention(
            q, cache.keys, cache.values, attended, ctx.query_start, ctx.seq_lens, group.block_table, None,
            nq, nkv, d, dv, group.page_size, self.scale, self.window, ctx.max_query_len, ctx.max_seq_len,
            ctx.num_decode, sinks=self.sinks, **gate)
        if not self.output_gate and factor != 1.0:
            if not attended.is_contiguous():
                raise ValueError("an ungated attention with a factor writes rows of its own")
            kernels.scaled_sum(attended, factor, attended, 0.0, attended)
        return attended

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        inner = self.forward_inner(x, ctx, cache)
        out = torch.empty((x.shape[0], self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(inner, self.out_proj, out)
        return out
