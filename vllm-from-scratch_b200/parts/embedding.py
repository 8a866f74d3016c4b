"""The two ends of the model: token ids into the residual stream, and normalised rows of
it into logits.

``token_embedding``: a row of the ``[vocab, hidden]`` table per token, widened to float32
(minivllm/models/qwen3.py:300-306).  ``linear_head``: logits = rows . W^T in float32, W
being the embedding's table when ``tied`` (minivllm/models/qwen3.py:372-376, 393-395).
Both are parts like any other: an architecture whose embedding is scaled, or whose logits
are capped, registers its own kinds and names them in its ``ModelSpec``.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import (EMBEDDINGS, OUTPUT_HEADS, CacheView, Embedding, OutputHead, PartEnv, StateNeed, StepContext,
                   WeightInfo)


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size``; ``weight_name`` (default ``weight``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.vocab_size = int(params["vocab_size"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        return {self.weight_name: WeightInfo((self.vocab_size, self.env.hidden_size))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, residual: torch.Tensor,
                error_flag: torch.Tensor) -> None:
        kernels.embedding(self.weight, token_ids, residual, error_flag)

    def table(self) -> torch.Tensor:
        return self.weight


@EMBEDDINGS.register("bigram_embedding")
class BigramEmbedding(Embedding):
    """A row per token plus a row per pair (previous token, token) from a hashed table: row
    ``(previous * mul_prev + token * mul_cur) mod buckets`` of ``bigram`` (``buckets + 1`` rows; the
    last one is for a sequence's first token).  The previous token is state of the request: the
    kernel reads it from the request's slot for the first token of a portion and leaves the
    portion's last token there.

    params: ``vocab_size``, ``buckets``, ``mul_prev``, ``mul_cur``; ``scale`` (the token's row is multiplied
    by it, the pair's row is not; default 1); ``weight_names`` (token table, bigram table; default
    ``weight``, ``bigram``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.vocab_size = int(params["vocab_size"])
        self.buckets = int(params["buckets"])
        self.mul_prev, self.mul_cur = int(params["mul_prev"]), int(params["mul_cur"])
        self.scale = float(params.get("scale", 1.0))
        if self.buckets <= 0:
            raise ValueError(f"bigram embedding: buckets={self.buckets}")
        self.names = tuple(params.get("weight_names", ("weight", "bigram")))
        self.weight: torch.Tensor | None = None
        self.bigram: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden = self.env.hidden_size
        return {self.names[0]: WeightInfo((self.vocab_size, hidden)),
                self.names[1]: WeightInfo((self.buckets + 1, hidden))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.names[0]].contiguous()
        self.bigram = tensors[self.names[1]].contiguous()

    def cache_need(self) -> StateNeed:
        return StateNeed((1,), torch.int32, name="previous_token")

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, residual: torch.Tensor,
                error_flag: torch.Tensor, cache: CacheView | None = None) -> None:
        if cache is None or cache.state is None:
            raise ValueError("the bigram embedding keeps the previous token per request: it needs its state")
        kernels.bigram_embedding(self.weight, self.bigram, token_ids, ctx.positions, ctx.token_request,
                                 ctx.query_start, ctx.state_slots, cache.state, residual, self.mul_prev,
                                 self.mul_cur, error_flag, scale=self.scale)

    def table(self) -> torch.Tensor:
        return self.weight


@OUTPUT_HEADS.register("linear_head")
class LinearHead(OutputHead):
    """params: ``vocab_size``, ``tied`` (default False), ``scale`` (the logits are multiplied by it;
    default 1), ``weight_name`` (default ``weight``; empty: the prefix itself is the tensor)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.vocab_size = int(params["vocab_size"])
        self.tied = bool(params.get("tied", False))
        self.scale = float(params.get("scale", 1.0))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        return {} if self.tied else {self.weight_name: WeightInfo((self.vocab_size, self.env.hidden_size))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def bind_embedding(self, embedding: Embedding) -> None:
        if self.tied:
            self.weight = embedding.table()         # the very tensor: read once a step, held once

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        out = torch.empty((normed.shape[0], self.vocab_size), dtype=torch.float32, device=normed.device)
        kernels.gemm(normed, self.weight, out)
        if self.scale != 1.0:
            out.mul_(self.scale)        # float32, one rounding per logit
        return out
