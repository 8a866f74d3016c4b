"""Python face of the kernels for products in groups (a matrix per expert, a matrix per head), for
routing tokens to experts, and for the gated activations that go with them (``csrc/grouped.cu``).

As everywhere in this package there is no CPU or library alternative behind these functions.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _F, _I, _P, KernelError, _check, _code, _run, _stream

_RUN = (torch.float32, torch.bfloat16)
_L = ctypes.c_longlong

GATE_NONE, GATE_SILU, GATE_CAPPED = 0, 1, 2


def route_experts(x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, ids: torch.Tensor,
                  weights: torch.Tensor, top: int, group_count: int = 1, group_keep: int = 1,
                  group_top: int = 2, scoring: str = "sigmoid", renormalise: bool = False) -> None:
    """For every row of ``x`` ``[T, K]``: logits ``router @ x`` in float32 (``router`` float32 ``[E, K]``),
    scores = sigmoid of each (``scoring="softmax"``: the softmax over all E of them; ``renormalise``: the
    weights are the chosen scores divided by their sum + 1e-20); the ``top`` experts with the largest ``score + correction`` among the experts of
    the ``group_keep`` best of ``group_count`` equal groups of neighbours (a group's mark: the sum of its
    ``group_top`` largest ``score + correction``) go to ``ids`` (int32 ``[T, top]``), their plain scores
    to ``weights`` (float32 ``[T, top]``).  Ties go to the smaller index."""
    tokens, k = x.shape
    experts = router.shape[0]
    if scoring not in ("sigmoid", "softmax"):
        raise KernelError(f"router scores {scoring!r}: 'sigmoid' or 'softmax'")
    _run("grouped", "b200_route_experts",
         _P(_check("router input", x, _RUN)), _P(_check("router matrix", router, torch.float32, (experts, k))),
         _P(_check("score correction", correction, torch.float32, (experts,), optional=True)),
         _P(_check("chosen experts", ids, torch.int32, (tokens, top))),
         _P(_check("weights of the chosen", weights, torch.float32, (tokens, top))),
         _I(tokens), _I(k), _I(experts), _I(top), _I(group_count), _I(group_keep), _I(group_top),
         _I(1 if scoring == "softmax" else 0), _I(1 if renormalise else 0), _I(_code(x.dtype)), _stream())


def expert_lists(ids: torch.Tensor, experts: int, offsets: torch.Tensor, sorted_pair: torch.Tensor,
                 position: torch.Tensor) -> None:
    """From ``ids`` (int32 ``[T, top]``): ``offsets`` (int32 ``[experts + 1]``) where each expert's rows
    begin, ``sorted_pair`` (int32 ``[T * top]``) the pairs ``token * top + choice`` expert by expert, and
    ``position`` (int32 ``[T * top]``) the row of each pair."""
    pairs = ids.numel()
    _run("grouped", "b200_expert_lists", _P(_check("chosen experts", ids, torch.int32)), _I(pairs), _I(experts),
         _P(_check("list offsets", offsets, torch.int32, (experts + 1,))),
         _P(_check("sorted pairs", sorted_pair, torch.int32, (pairs,))),
         _P(_check("rows of the pairs", position, torch.int32, (pairs,))), _stream())


def gather_rows(x: torch.Tensor, index: torch.Tensor, divisor: int, out: torch.Tensor) -> None:
    """``out[r] = x[index[r] // divisor]``."""
    rows, width = out.shape
    _run("grouped", "b200_gather_rows", _P(_check("rows to gather from", x, _RUN, (None, width))),
         _P(_check("row index", index, torch.int32, (rows,))), _I(divisor), _P(_check("gathered rows", out, x.dtype)),
         _I(rows), _I(width), _I(_code(x.dtype)), _stream())


def combine_experts(rows: torch.Tensor, position: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor,
                    identity: tuple[torch.Tensor, torch.Tensor, int] | None = None,
                    extra: torch.Tensor | None = None, top: int | None = None) -> None:
    """``out[t] = sum_j weights[t, j] * rows[position[t * top + j]]`` in float32, j in order (a pair whose
    position is negative adds nothing).  ``identity = (ids, x, experts)``: a pair whose expert number ``ids[t, j]``
    is ``experts`` or more belongs to an identity expert and adds ``weights[t, j] * x[t]``.  ``extra`` ``[T,
    width]``: rows added to every token's sum (an expert that every token passes).  ``weights`` None (with
    ``top``, the choices a token has): every weight is 1, for experts whose weight went into their input."""
    tokens, width = out.shape
    if weights is None and top is None:
        raise KernelError("combine_experts: without weights, say how many choices a token has (top=)")
    top = weights.shape[1] if weights is not None else int(top)
    ids = x = experts = 0
    if identity is not None:
        ids = _check("chosen experts", identity[0], torch.int32, (tokens, top))
        x = _check("expert input", identity[1], out.dtype, (tokens, width))
        experts = int(identity[2])
    _run("grouped", "b200_combine_experts", _P(_check("expert rows", rows, out.dtype, (None, width))),
         _P(_check("rows of the pairs", position, torch.int32, (tokens * top,))),
         _P(_check("weights", weights, torch.float32, (tokens, top), optional=True)),
         _P(_check("combined output", out, _RUN)),
         _I(tokens), _I(width), _I(top), _P(ids), _P(x), _I(experts),
         _P(_check("rows added to every sum", extra, out.dtype, (tokens, width), optional=True)),
         _I(_code(out.dtype)), _stream())


def _gate(gated) -> tuple[int, float, float, float]:
    if gated is None:
        return GATE_NONE, 0.0, 0.0, 0.0
    if gated == "silu":
        return GATE_SILU, 0.0, 0.0, 0.0
    kind, limit, slope, offset = gated
    if kind != "capped":
        raise KernelError(f"gated epilogue {gated!r}: 'silu' or ('capped', limit, slope, offset)")
    return GATE_CAPPED, float(limit), float(slope), float(offset)


def expert_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor,
                row_index: torch.Tensor | None, index_divisor: int = 1, gated=None,
                row_scale: torch.Tensor | None = None) -> None:
    """Rows in lists, a matrix per list: for list e (rows ``offsets[e]`` to ``offsets[e + 1]``) ``out[row] =
    x[source(row)] @ w[e]^T``; ``source(row) = row_index[row] // index_divisor`` or, without an index,
    the row itself.  ``w`` is ``[E, N, K]``; ``gated``: ``w`` is ``[E, 2 N, K]`` with the gate rows first and
    ``out = act(gate) * up``: ``"silu"``, or ``("capped", limit, slope, offset)`` for ``g sigmoid(slope g) (u +
    offset)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``.  ``row_scale`` (float32): the products
    of a row are multiplied by ``row_scale[row_index[row]]`` (without an index: ``row_scale[row]``) ahead of their
    rounding and of the activation, which is the expert given ``scale * x`` in place of ``x``."""
    experts, wn, k = w.shape
    list_rows, n = out.shape
    kind, limit, slope, offset = _gate(gated)
    if wn != (2 * n if kind else n):
        raise KernelError(f"expert matrices {tuple(w.shape)} do not give {n} columns")
    _run("grouped", "b200_grouped_gemm_scaled",
         _P(_check("expert input", x, _RUN, (None, k))), _P(_check("expert matrices", w, x.dtype)),
         _P(_check("expert output", out, x.dtype)), _P(_check("list offsets", offsets, torch.int32, (experts + 1,))),
         _P(_check("row index", row_index, torch.int32, (list_rows,), optional=True)), _I(index_divisor), _I(0),
         _I(list_rows), _I(experts), _I(n), _I(k), _L(k), _L(n), _L(0), _L(0), _I(kind), _F(limit), _F(slope),
         _F(offset), _P(_check("row factors", row_scale, torch.float32, optional=True)), _I(_code(x.dtype)), _stream())


def head_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, column: int = 0) -> None:
    """A matrix per head: rows of ``x`` hold the heads' inputs side by side (``K`` columns each, the first
    at ``column`` of a possibly wider row), rows of ``out`` ``[T, H * N]`` their outputs: ``out[t, h] = x[t, h]
    @ w[h]^T`` with ``w`` ``[H, N, K]``."""
    heads, n, k = w.shape
    tokens, stride = x.shape
    if column < 0 or column + heads * k > stride:
        raise KernelError(f"head inputs: columns {column} to {column + heads * k} of rows of {stride}")
    _check("head inputs", x, _RUN)
    _run("grouped", "b200_grouped_gemm",
         _P(x.data_ptr() + column * x.element_size()), _P(_check("head matrices", w, x.dtype)),
         _P(_check("head outputs", out, x.dtype, (tokens, heads * n))), _P(0), _P(0), _I(1), _I(tokens), _I(0),
         _I(heads), _I(n), _I(k), _L(stride), _L(heads * n), _L(k), _L(n), _I(0), _F(0.0), _F(0.0), _F(0.0),
         _I(_code(x.dtype)), _stream())


def capped_swish_mul(gate_up: torch.Tensor, out: torch.Tensor, limit: float | None, slope: float,
                     offset: float, row_scale: torch.Tensor | None = None,
                     row_index: torch.Tensor | None = None) -> None:
    """``out = g * sigmoid(slope * g) * (u + offset)`` in float32 with ``g = min(gate_up[:, :I], limit)`` and
    ``u = clamp(gate_up[:, I:], -limit, limit)`` (``limit`` None: no cap).  ``row_scale`` (float32): row r of
    ``gate_up`` is multiplied by ``row_scale[row_index[r]]`` (without an index: ``row_scale[r]``) ahead of the caps."""
    tokens, inter = out.shape
    _run("grouped", "b200_capped_swish_mul_scaled", _P(_check("gate_up", gate_up, out.dtype, (tokens, 2 * inter))),
         _P(_check("activation output", out, _RUN)), _I(tokens), _I(inter),
         _F(math.inf if limit is None else limit), _F(slope), _F(offset),
         _P(_check("row factors", row_scale, torch.float32, optional=True)),
         _P(_check("rows of the factors", row_index, torch.int32, optional=True)), _I(_code(out.dtype)), _stream())


def gelu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = gelu_tanh(gate_up[:, :I]) * gate_up[:, I:]`` in float32, with ``gelu_tanh(z) = z / 2 * (1 +
    tanh(sqrt(2 / pi) * (z + 0.044715 z^3)))``."""
    tokens, inter = out.shape
    _run("grouped", "b200_gelu_mul", _P(_check("gate_up", gate_up, out.dtype, (tokens, 2 * inter))),
         _P(_check("activation output", out, _RUN)), _I(tokens), _I(inter), _I(_code(out.dtype)), _stream())


def gelu_gate_rows(gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
                   column: int) -> None:
    """``out[t] = gelu_tanh(gate[t]) * table[ids[t], column : column + dim]`` in float32."""
    tokens, dim = gate.shape
    vocab, stride = table.shape
    _run("grouped", "b200_gelu_gate_rows", _P(_check("gate rows", gate, _RUN)),
         _P(_check("table", table, gate.dtype)), _P(_check("token ids", ids, torch.int32, (tokens,))),
         _P(_check("gated rows", out, gate.dtype, (tokens, dim))), _I(tokens), _I(dim), _I(stride), _I(column),
         _I(vocab), _I(_code(gate.dtype)), _stream())
