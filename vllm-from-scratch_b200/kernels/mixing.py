"""Python face of the kernels for mixers beyond rotary softmax attention and for the norm forms
that go with them: attention with a distance bias and keys and values of sizes of their own,
recurrences with a matrix of state per head (decayed linear attention, selective scan), the short
causal convolution, norms with a second operand, and the embedding with a bigram table.

As everywhere in this package there is no CPU or library alternative behind these functions.
"""

from __future__ import annotations

import ctypes

import torch

from . import _F, _I, _P, _check, _code, _run, _stream, count_launch

_RUN = (torch.float32, torch.bfloat16)


# ------------------------------------------------------------------------ norms
def add_normed_rmsnorm(x: torch.Tensor | None, x_weight: torch.Tensor | None, x_eps: float, residual: torch.Tensor,
                       weight: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                       rows: torch.Tensor | None = None) -> None:
    """``residual += rms(x) * x_weight`` in float32 (skipped when ``x`` is None), then ``out =
    rms(residual) * weight`` in ``out``'s dtype; ``weight`` None: ``out`` is the residual itself in
    ``out``'s dtype (what a sublayer reads that has no norm in front of it); ``out`` None as well:
    the sum only.  With ``rows`` only those rows are formed, written compactly to ``out``, and
    ``residual`` is left as it was."""
    tokens, hidden = residual.shape
    out_rows = tokens if rows is None else rows.shape[0]
    dtype = x.dtype if x is not None else out.dtype
    _run("norm_ext", "b200_add_normed_rmsnorm",
         _P(_check("normed addend", x, _RUN, (tokens, hidden), optional=True)),
         _P(_check("addend norm weight", x_weight, torch.float32, (hidden,), optional=True)), _F(x_eps),
         _P(_check("residual", residual, torch.float32)),
         _P(_check("norm weight", weight, torch.float32, (hidden,), optional=True)),
         _P(_check("norm output", out, dtype, (out_rows, hidden), optional=True)),
         _P(_check("row index", rows, torch.int32, optional=True)),
         _I(out_rows), _I(hidden), _F(eps), _I(_code(dtype)), _stream())


def paired_norm_mean(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float,
                     out: torch.Tensor) -> None:
    """``out = (rms(a) * wa + rms(b) * wb) / 2`` row by row, in float32."""
    tokens, hidden = a.shape
    _run("norm_ext", "b200_paired_norm_mean",
         _P(_check("first branch", a, _RUN, (tokens, hidden))), _P(_check("first weight", wa, torch.float32, (hidden,))),
         _P(_check("second branch", b, a.dtype, (tokens, hidden))), _P(_check("second weight", wb, torch.float32, (hidden,))),
         _P(_check("mean output", out, a.dtype, (tokens, hidden))), _I(tokens), _I(hidden), _F(eps),
         _I(_code(a.dtype)), _stream())


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, groups: int,
                     gate_first: bool, eps: float, silu_behind: bool = False) -> None:
    """``y`` float32 ``[T, W]``; ``gate`` rows whose first W elements are the gate (a view of a
    wider projection will do: only its row stride is used); ``out`` may be a view of ``W`` columns of wider rows.
    ``gate_first``: ``out = rms_g(y *
    silu(gate)) * weight``; otherwise ``out = rms_g(y) * weight * sigmoid(gate)`` (``silu_behind``:
    ``* silu(gate)``); ``rms_g`` normalises each of ``groups`` equal parts of a row by its own root
    mean square."""
    if gate_first and silu_behind:
        from . import KernelError
        raise KernelError("gated_group_norm: the gate is either ahead of the norm or behind it")
    tokens, width = y.shape
    _check("recurrence output", y, torch.float32)
    _check("gated norm weight", weight, torch.float32, (width,))
    if (not out.is_cuda or out.dtype not in _RUN or tuple(out.shape) != (tokens, width) or out.stride(1) != 1
            or out.stride(0) < width):
        from . import KernelError
        raise KernelError(f"gated norm output: shape {tuple(out.shape)}, strides {out.stride()}, dtype {out.dtype}")
    if gate.dtype != out.dtype or gate.dim() != 2 or gate.shape[0] != tokens or gate.shape[1] < width \
            or gate.stride(1) != 1 or not gate.is_cuda:
        from . import KernelError
        raise KernelError(f"gate: shape {tuple(gate.shape)}, strides {gate.stride()}, dtype {gate.dtype}")
    _run("norm_ext", "b200_gated_group_norm_rows", _P(y.data_ptr()), _P(gate.data_ptr()), _I(gate.stride(0)),
         _P(weight.data_ptr()), _P(out.data_ptr()), _I(out.stride(0)), _I(tokens), _I(width), _I(groups),
         _I(1 if gate_first else 2 if silu_behind else 0),
         _F(eps), _I(_code(out.dtype)), _stream())


def bigram_embedding(table: torch.Tensor, bigram: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                     token_request: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor,
                     previous: torch.Tensor, residual: torch.Tensor, mul_prev: int, mul_cur: int,
                     error_flag: torch.Tensor, scale: float = 1.0) -> None:
    """``residual[t] = table[ids[t]] * scale + bigram[(before * mul_prev + ids[t] * mul_cur) mod buckets]`` in
    float32, ``before`` being the token ahead of t in its request: the one in this step, or, for a
    portion's first token, ``previous[slot]``; a sequence's first token takes the table's last row.
    ``previous`` (int32 ``[slots + 1, 1]``) then holds every request's last token."""
    vocab, hidden = table.shape
    tokens = ids.shape[0]
    buckets = bigram.shape[0] - 1
    requests = slots.shape[0]
    _run("norm_ext", "b200_bigram_embedding",
         _P(_check("embedding table", table, _RUN)), _P(_check("bigram table", bigram, table.dtype, (buckets + 1, hidden))),
         _P(_check("token ids", ids, torch.int32, (tokens,))), _P(_check("positions", positions, torch.int32, (tokens,))),
         _P(_check("request of each token", token_request, torch.int32, (tokens,))),
         _P(_check("query_start", query_start, torch.int32, (requests + 1,))),
         _P(_check("state slots", slots, torch.int32, (requests,))),
         _P(_check("previous tokens", previous, torch.int32)),
         _P(_check("residual", residual, torch.float32, (tokens, hidden))),
         _I(tokens), _I(hidden), _I(vocab), _I(buckets), _I(mul_prev), _I(mul_cur), _F(scale),
         _P(_check("error flag", error_flag, torch.int32)), _I(_code(table.dtype)), _stream())


# -------------------------------------------------------------------- attention
def head_norm_scale_cache(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                          q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                          temperature: tuple[float, int] | None, q_out: torch.Tensor,
                          k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, num_q_heads: int,
                          num_kv_heads: int, head_dim: int, value_dim: int, page_size: int,
                          unit_norm: bool = False, column: int = 0) -> None:
    """From the packed projection ``[T, nq d + nkv d + nkv dv]``: per-head RMSNorm of queries and
    keys, queries times ``1 + coef * ln(floor((p + 1) / every) + 1)`` for ``temperature = (coef,
    every)``, queries to ``q_out``, keys and values to their pages at ``slots``.

    ``unit_norm``: queries and keys are divided by their root mean square also where no weight
    vector is given (without it an absent weight means no norm).  ``value_dim = 0``: keys only, no
    values are stored (``num_q_heads = 0`` with it: rows of keys alone are normalised into their
    pages).  ``column``: the rows begin at that column of a wider ``qkv``."""
    tokens = qkv.shape[0]
    dtype = qkv.dtype
    width = (num_q_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim
    coef, every = temperature if temperature is not None else (0.0, 0)
    stride = qkv.shape[1]
    if column < 0 or column + width > stride:
        from . import KernelError
        raise KernelError(f"qkv: columns {column} to {column + width} of rows of {stride}")
    _check("qkv", qkv, _RUN, (tokens, stride))
    _run("attention_bias", "b200_head_norm_scale_cache",
         _P(qkv.data_ptr() + column * qkv.element_size()),
         _P(_check("positions", positions, torch.int32, (tokens,))),
         _P(_check("slot mapping", slots, torch.int32, (tokens,))),
         _P(_check("q head-norm weight", q_weight, torch.float32, (head_dim,), optional=True)),
         _P(_check("k head-norm weight", k_weight, torch.float32, (head_dim,), optional=True)),
         _P(_check("q output", q_out, dtype, (tokens, num_q_heads * head_dim), optional=num_q_heads == 0)),
         _P(_check("key pages", k_pages, dtype, (None, num_kv_heads, page_size, head_dim), optional=True)),
         _P(_check("value pages", v_pages, dtype, (None, num_kv_heads, page_size, value_dim), optional=True)
            if value_dim else 0),
         _I(tokens), _I(num_q_heads), _I(num_kv_heads), _I(head_dim), _I(value_dim), _I(page_size),
         _F(eps), _F(coef), _I(every), _I(stride), _I(1 if (unit_norm or q_weight is not None) else 0),
         _I(1 if (unit_norm or k_weight is not None) else 0), _I(_code(dtype)), _stream())


NORM_KINDS = {None: 0, "head": 1, "whole": 2}


def qk_prepare_cache(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor,
                     q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, norm: str | None, eps: float,
                     inv_freq: torch.Tensor | None, rotary_dim: int, interleaved: bool, q_out: torch.Tensor,
                     k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, num_q_heads: int,
                     num_kv_heads: int, head_dim: int, value_dim: int, page_size: int) -> None:
    """From the first ``nq d + nkv d + nkv dv`` columns of the projection's rows: ``bias`` added (float32, that
    many numbers), RMSNorm of queries and keys (``norm``: None, ``"head"`` with weight vectors of ``d`` numbers for
    all heads, ``"whole"`` over all heads of q and of k at once with weight vectors of ``nq d`` and ``nkv d``
    numbers; a weight may be None), rotation of the first ``rotary_dim`` numbers of every query and key head by the
    angles ``position * inv_freq[i]`` (``interleaved``: the pairs are neighbours ``(2i, 2i + 1)``, else halves
    ``(i, i + rotary_dim / 2)``), queries to ``q_out``, keys and values to their pages at ``slots``.  ``num_kv_heads
    = 0``: rows of queries alone (a layer that reads another layer's pages)."""
    tokens, stride = qkv.shape
    dtype = qkv.dtype
    width = (num_q_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim
    if norm not in NORM_KINDS:
        from . import KernelError
        raise KernelError(f"qk_prepare_cache: norm {norm!r} (None, 'head' or 'whole')")
    q_size = (head_dim,) if norm == "head" else (num_q_heads * head_dim,)
    k_size = (head_dim,) if norm == "head" else (num_kv_heads * head_dim,)
    store = num_kv_heads > 0 and k_pages is not None
    _run("qk_prepare", "b200_qk_prepare_cache",
         _P(_check("qkv", qkv, _RUN)), _P(_check("projection bias", bias, torch.float32, (width,), optional=True)),
         _P(_check("positions", positions, torch.int32, (tokens,))),
         _P(_check("slot mapping", slots, torch.int32, (tokens,))),
         _P(_check("q norm weight", q_weight, torch.float32, q_size, optional=True)),
         _P(_check("k norm weight", k_weight, torch.float32, k_size, optional=True)),
         _P(_check("inverse frequencies", inv_freq, torch.float32, (rotary_dim // 2,), optional=True)),
         _P(_check("q output", q_out, dtype, (tokens, num_q_heads * head_dim))),
         _P(_check("key pages", k_pages, dtype, (None, num_kv_heads, page_size, head_dim)) if store else 0),
         _P(_check("value pages", v_pages, dtype, (None, num_kv_heads, page_size, value_dim)) if store else 0),
         _I(tokens), _I(num_q_heads), _I(num_kv_heads), _I(head_dim), _I(value_dim), _I(page_size), _I(stride),
         _I(NORM_KINDS[norm]), _I(rotary_dim if inv_freq is not None else 0), _I(1 if interleaved else 0), _F(eps),
         _I(_code(dtype)), _stream())


def head_gate(x: torch.Tensor, gate: torch.Tensor, gate_column: int, out: torch.Tensor, heads: int,
              factor: float = 1.0) -> None:
    """``out[t, h, :] = x[t, h, :] * sigmoid(gate[t, gate_column + h]) * factor`` in float32; ``gate`` may be a
    wider projection of which ``heads`` columns from ``gate_column`` on are the gates.  ``out`` may be ``x``."""
    tokens, width = x.shape
    if gate.dim() != 2 or gate.shape[0] != tokens or gate_column < 0 or gate_column + heads > gate.shape[1] or width % heads:
        from . import KernelError
        raise KernelError(f"head_gate: {heads} gates at column {gate_column} of rows {tuple(gate.shape)} for {tuple(x.shape)}")
    _check("gate rows", gate, x.dtype)
    _run("qk_prepare", "b200_head_gate", _P(_check("heads' outputs", x, _RUN)),
         _P(gate.data_ptr() + gate_column * gate.element_size()), _I(gate.shape[1]),
         _P(_check("gated outputs", out, x.dtype, (tokens, width))), _I(tokens), _I(heads), _I(width // heads),
         _F(factor), _I(_code(x.dtype)), _stream())


def scaled_sum(a: torch.Tensor, scale_a: float, b: torch.Tensor, scale_b: float, out: torch.Tensor) -> None:
    """``out = a * scale_a + b * scale_b`` element by element, in float32."""
    _run("qk_prepare", "b200_scaled_sum", _P(_check("first addend", a, _RUN)), _F(scale_a),
         _P(_check("second addend", b, a.dtype, tuple(a.shape))), _F(scale_b),
         _P(_check("sum", out, a.dtype, tuple(a.shape))), ctypes.c_longlong(a.numel()), _I(_code(a.dtype)), _stream())


# Tests set this to False to drive the float32-arithmetic kernel through the same call.
USE_TENSOR_CORES = True
_sms: dict = {}


def _sm_count() -> int:
    device = torch.cuda.current_device()
    if device not in _sms:
        from ..csrc.build import load_library
        _sms[device] = int(load_library("attention_bias").b200_biased_sm_count()) or 1
    return _sms[device]


def biased_paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                           query_start: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                           slopes: torch.Tensor | None, num_q_heads: int, num_kv_heads: int, head_dim: int,
                           value_dim: int, page_size: int, scale: float, window: int | None,
                           max_query_len: int | None = None, max_seq_len: int | None = None,
                           num_decode: int = 0, sinks: torch.Tensor | None = None,
                           gate: torch.Tensor | None = None, gate_column: int = 0, gate_factor: float = 1.0) -> None:
    """Causal attention of every request's new queries over its pages with the score ``q . k * scale
    - slopes[h] * (i - j)``; scores, weights and the weighted sum in float32.  ``sinks`` (float32, one
    per query head): ``exp(sinks[h])`` joins the softmax denominator of head h once, unscaled, with no
    key and no value.  ``v_pages`` may be ``k_pages`` itself (keys that serve as the values too).
    ``gate`` (rows of the run dtype, a number per query head from ``gate_column`` on; a wider projection will do):
    head h's output is multiplied by ``gate_factor * sigmoid(gate[t, gate_column + h])`` as it is written.
    ``out`` may be a view of the first ``nq * dv`` columns of wider rows (the heads of another mixer behind them).

    bfloat16 with keys and values of one size of 64, 128 or 256 (and ``max_query_len`` and
    ``max_seq_len`` given): the tensor-core kernels, whose softmax weights enter the second product
    as three bfloat16 pieces that add up to the float32 weight; requests that bring one token (all
    of them when ``max_query_len`` is 1, else the first ``num_decode``) go to the kernel that splits
    the keys over blocks, portions to the 64-row kernel.  Everything else: one kernel in float32
    arithmetic."""
    tokens = q.shape[0]
    requests = seq_lens.shape[0]
    dtype = q.dtype
    checked = (
        _check("queries", q, _RUN, (tokens, num_q_heads * head_dim)),
        _check("key pages", k_pages, dtype, (None, num_kv_heads, page_size, head_dim)),
        _check("value pages", v_pages, dtype, (None, num_kv_heads, page_size, value_dim)),
        out.data_ptr(),
        _check("query_start", query_start, torch.int32, (requests + 1,)),
        _check("seq_lens", seq_lens, torch.int32, (requests,)),
        _check("block table", block_table, torch.int32, (requests, None)),
        _check("slopes", slopes, torch.float32, (num_q_heads,), optional=True),
        _check("sinks", sinks, torch.float32, (num_q_heads,), optional=True))
    if (not out.is_cuda or out.dtype != dtype or tuple(out.shape) != (tokens, num_q_heads * value_dim)
            or (out.stride(1) != 1 and out.shape[1] > 1) or out.stride(0) < out.shape[1]):
        from . import KernelError
        raise KernelError(f"attention output: shape {tuple(out.shape)}, strides {out.stride()}, dtype {out.dtype}")
    out_stride = 0 if out.is_contiguous() else out.stride(0)
    gate_p, gate_stride = 0, 0
    if gate is not None:
        if (gate.dtype != dtype or gate.dim() != 2 or gate.shape[0] != tokens or not gate.is_contiguous()
                or gate_column < 0 or gate_column + num_q_heads > gate.shape[1]):
            from . import KernelError
            raise KernelError(f"gates: {num_q_heads} columns from {gate_column} of rows {tuple(gate.shape)}, dtype {gate.dtype}")
        gate_p, gate_stride = gate.data_ptr() + gate_column * gate.element_size(), gate.shape[1]
    form = (_P(gate_p), _I(gate_stride), _F(gate_factor), _I(out_stride))
    # The decode kernel takes up to 16 query heads on a key/value head; more run as several groups that
    # read the same cached head.
    launch_kv = next(m for m in range(num_kv_heads, num_q_heads + 1, num_kv_heads)
                     if num_q_heads % m == 0 and (num_q_heads // m <= 16 or m == num_q_heads))
    if (USE_TENSOR_CORES and dtype == torch.bfloat16 and max_query_len is not None and max_seq_len is not None
            and head_dim == value_dim and head_dim in (64, 128, 256) and num_q_heads % launch_kv == 0
            and num_q_heads // launch_kv <= 16 and out_stride % 2 == 0):
        from .attention_bf16 import decode_splits
        cached_heads, num_kv_heads = num_kv_heads, launch_kv
        q_p, k_p, v_p, out_p, start_p, lens_p, table_p, slopes_p, sinks_p = checked
        single = requests if (max_query_len == 1 and tokens == requests) else num_decode
        width = block_table.shape[1]
        if single > 0:
            splits = decode_splits(single, num_kv_heads, max_seq_len, _sm_count())
            partial_o = partial_ml = None
            if splits > 1:
                partial_o = torch.empty((single * num_q_heads * splits, head_dim), dtype=torch.float32, device=q.device)
                partial_ml = torch.empty((single * num_q_heads * splits, 2), dtype=torch.float32, device=q.device)
            _run("attention_bias", "b200_biased_decode_attention_bf16", _P(q_p), _P(k_p), _P(v_p), _P(out_p),
                 _P(partial_o.data_ptr() if splits > 1 else 0), _P(partial_ml.data_ptr() if splits > 1 else 0),
                 _P(lens_p), _P(table_p), _P(slopes_p), _P(sinks_p), _I(single), _I(width), _I(num_q_heads), _I(num_kv_heads),
                 _I(head_dim), _I(page_size), _F(scale), _I(window or 0), _I(splits), _I(cached_heads), *form, _stream())
            if splits > 1:
                count_launch()
        if single < requests:
            # The requests behind the single tokens: their rows of the block table and of the lengths,
            # the batch's own q, out, gates and query_start (rows of the whole batch).
            _run("attention_bias", "b200_biased_prefill_attention_bf16", _P(q_p), _P(k_p), _P(v_p), _P(out_p),
                 _P(start_p + 4 * single), _P(lens_p + 4 * single), _P(table_p + 4 * single * width), _P(slopes_p),
                 _P(sinks_p),
                 _I(requests - single), _I(tokens), _I(width), _I(num_q_heads), _I(num_kv_heads), _I(head_dim),
                 _I(page_size), _F(scale), _I(window or 0), _I(single), _I(cached_heads), *form, _stream())
        return
    _run("attention_bias", "b200_biased_paged_attention",
         *(_P(address) for address in checked),
         _I(requests), _I(tokens), _I(block_table.shape[1]), _I(num_q_heads), _I(num_kv_heads), _I(head_dim),
         _I(value_dim), _I(page_size), _F(scale), _I(window or 0), *form, _I(_code(dtype)), _stream())


# ------------------------------------------------------------------ recurrences
# A portion of at least twice this many tokens is cut into segments of about this length that run
# side by side (see csrc/recurrence.cu); tests lower it to cut short sequences too.
SCAN_SEGMENT = 256
SCAN_SCRATCH_BYTES = 256 << 20      # the most that the segments' states may take


def _recurrence_sms() -> int:
    device = torch.cuda.current_device()
    if ("recurrence", device) not in _sms:
        from ..csrc.build import load_library
        _sms[("recurrence", device)] = int(load_library("recurrence").b200_recurrence_sm_count()) or 1
    return _sms[("recurrence", device)]


def _segments(max_query_len: int | None, requests: int, heads: int, rows: int, columns: int, device
              ) -> tuple[int, int, torch.Tensor | None, torch.Tensor | None]:
    """``(seg_len, segs, states, decays)`` for a step whose longest portion has ``max_query_len`` tokens;
    ``segs`` is 1 (and nothing is allocated) where the portions are short or the scratch would be too large."""
    if max_query_len is None or max_query_len < 2 * SCAN_SEGMENT:
        return 0, 1, None, None
    # Segments cost half as much work again (the second pass).  They pay where the launch would leave
    # most SMs without a block (a linear-attention layer of 8 heads: 385 against 194 us for 2048 tokens);
    # a launch that fills half of the GPU already is bound by its arithmetic and would only lose.
    if 2 * requests * heads * -(-columns // 32) > _recurrence_sms():
        return 0, 1, None, None
    per_segment = requests * heads * rows * columns * 4
    segs = min(-(-max_query_len // SCAN_SEGMENT), SCAN_SCRATCH_BYTES // max(1, per_segment))
    if segs < 2:
        return 0, 1, None, None
    seg_len = -(-max_query_len // segs)
    seg_len = -(-seg_len // 16) * 16                    # whole tiles of the kernel
    segs = -(-max_query_len // seg_len)
    states = torch.empty((requests * segs, heads, rows, columns), dtype=torch.float32, device=device)
    decays = torch.empty((requests * segs, heads), dtype=torch.float32, device=device)
    return seg_len, segs, states, decays


def decayed_linear_attention(proj: torch.Tensor, offsets: tuple[int, int, int], decay: torch.Tensor,
                             query_start: torch.Tensor, slots: torch.Tensor, state: torch.Tensor,
                             y: torch.Tensor, heads: int, key_dim: int, value_dim: int,
                             max_query_len: int | None = None) -> None:
    """Per request and head, token after token: ``S <- decay_h S + k v^T``, ``y = S^T q`` with q, k
    (``heads x key_dim``) and v (``heads x value_dim``) = silu of the columns of ``proj`` that start
    at ``offsets = (q, k, v)``.  ``state``: float32 ``[slots + 1, heads, key_dim, value_dim]``, read
    at the request's slot and left advanced; ``y``: float32 ``[T, heads * value_dim]``.  With
    ``max_query_len`` (the longest portion of the step) long portions run in segments side by side."""
    tokens, stride = proj.shape
    requests = slots.shape[0]
    seg_len, segs, seg_state, seg_decay = _segments(max_query_len, requests, heads, key_dim, value_dim, proj.device)
    if segs > 1:
        count_launch(2)
    _run("recurrence", "b200_decayed_linear_attention",
         _P(_check("projection", proj, _RUN)), _I(stride), _I(offsets[0]), _I(offsets[1]), _I(offsets[2]),
         _P(_check("decay", decay, torch.float32, (heads,))),
         _P(_check("query_start", query_start, torch.int32, (requests + 1,))),
         _P(_check("state slots", slots, torch.int32, (requests,))),
         _P(_check("state", state, torch.float32, (None, heads, key_dim, value_dim))),
         _P(_check("recurrence output", y, torch.float32, (tokens, heads * value_dim))),
         _I(tokens), _I(requests), _I(heads), _I(key_dim), _I(value_dim), _I(seg_len), _I(segs),
         _P(seg_state.data_ptr() if segs > 1 else 0), _P(seg_decay.data_ptr() if segs > 1 else 0),
         _I(_code(proj.dtype)), _stream())


def gated_linear_attention(proj: torch.Tensor, offsets: tuple[int, int, int], gate: torch.Tensor, gate_offset: int,
                           gate_bias: torch.Tensor | None, tau: float, q_scale: float, query_start: torch.Tensor,
                           slots: torch.Tensor, state: torch.Tensor, y: torch.Tensor, heads: int, key_dim: int,
                           value_dim: int, max_query_len: int | None = None) -> None:
    """Per request and head, token after token: ``S <- diag(a) S + k v^T``, ``y = S^T (q * q_scale)`` with q, k
    (``heads x key_dim``) and v (``heads x value_dim``) the columns of ``proj`` that start at ``offsets = (q, k,
    v)``, as projected, and a decay per head and key channel ``a = sigmoid(z) ** (1 / tau)``, ``z`` = the columns
    ``gate_offset .. gate_offset + heads * key_dim`` of ``gate`` plus ``gate_bias`` (float32), formed in float32.
    ``state``: float32 ``[slots + 1, heads, key_dim, value_dim]``, read at the request's slot and left advanced;
    ``y``: float32 ``[T, heads * value_dim]``.  With ``max_query_len`` (the longest portion of the step) long
    portions run in segments side by side."""
    tokens, stride = proj.shape
    requests = slots.shape[0]
    seg_len, segs, seg_state, _ = _segments(max_query_len, requests, heads, key_dim, value_dim, proj.device)
    seg_decay = None
    if segs > 1:
        seg_decay = torch.empty((requests * segs, heads, key_dim), dtype=torch.float32, device=proj.device)
        count_launch(2)
    if tau <= 0:
        from . import KernelError
        raise KernelError(f"gated linear attention: tau={tau} must be positive")
    _run("recurrence", "b200_gated_linear_attention",
         _P(_check("projection", proj, _RUN)), _I(stride), _I(offsets[0]), _I(offsets[1]), _I(offsets[2]),
         _P(_check("decay logits", gate, proj.dtype, (tokens, None))), _I(gate.shape[1]), _I(gate_offset),
         _P(_check("decay bias", gate_bias, torch.float32, (heads * key_dim,), optional=True)),
         _F(1.0 / tau), _F(q_scale),
         _P(_check("query_start", query_start, torch.int32, (requests + 1,))),
         _P(_check("state slots", slots, torch.int32, (requests,))),
         _P(_check("state", state, torch.float32, (None, heads, key_dim, value_dim))),
         _P(_check("recurrence output", y, torch.float32, (tokens, heads * value_dim))),
         _I(tokens), _I(requests), _I(heads), _I(key_dim), _I(value_dim), _I(seg_len), _I(segs),
         _P(seg_state.data_ptr() if segs > 1 else 0), _P(seg_decay.data_ptr() if segs > 1 else 0),
         _I(_code(proj.dtype)), _stream())


def selective_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_offset: int, dt_bias: torch.Tensor,
                   a_log: torch.Tensor, skip: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor,
                   state: torch.Tensor, y: torch.Tensor, heads: int, groups: int, state_dim: int,
                   value_dim: int, max_query_len: int | None = None) -> None:
    """Per request and head, token after token, with ``dt = softplus(proj[t, dt_offset + h] +
    dt_bias[h])``: ``S <- exp(-exp(a_log_h) dt) S + dt B x^T``, ``y = S^T C + skip_h x``; x, B and C are
    the columns ``[heads * value_dim | groups * state_dim | groups * state_dim]`` of the float32
    ``xbc``.  ``state``: float32 ``[slots + 1, heads, state_dim, value_dim]``."""
    tokens = xbc.shape[0]
    requests = slots.shape[0]
    width = heads * value_dim + 2 * groups * state_dim
    seg_len, segs, seg_state, seg_decay = _segments(max_query_len, requests, heads, state_dim, value_dim, xbc.device)
    if segs > 1:
        count_launch(2)
    _run("recurrence", "b200_selective_scan",
         _P(_check("convolved inputs", xbc, torch.float32, (tokens, width))), _I(width),
         _P(_check("projection", proj, _RUN, (tokens, None))), _I(proj.shape[1]), _I(dt_offset),
         _P(_check("dt bias", dt_bias, torch.float32, (heads,))), _P(_check("A_log", a_log, torch.float32, (heads,))),
         _P(_check("skip", skip, torch.float32, (heads,))),
         _P(_check("query_start", query_start, torch.int32, (requests + 1,))),
         _P(_check("state slots", slots, torch.int32, (requests,))),
         _P(_check("state", state, torch.float32, (None, heads, state_dim, value_dim))),
         _P(_check("recurrence output", y, torch.float32, (tokens, heads * value_dim))),
         _I(tokens), _I(requests), _I(heads), _I(groups), _I(state_dim), _I(value_dim), _I(seg_len), _I(segs),
         _P(seg_state.data_ptr() if segs > 1 else 0), _P(seg_decay.data_ptr() if segs > 1 else 0),
         _I(_code(proj.dtype)), _stream())


def causal_conv_silu(proj: torch.Tensor, offset: int, weight: torch.Tensor, bias: torch.Tensor,
                     state: torch.Tensor, token_request: torch.Tensor, query_start: torch.Tensor,
                     slots: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, c] = silu(bias[c] + sum_i weight[i, c] * in[t - (taps - 1 - i), c])`` over the columns
    ``offset .. offset + channels`` of ``proj``, within each request (``weight`` is ``[taps, channels]``:
    a checkpoint's ``[channels, taps]`` transposed, the last row for the current token); what lies before a step's
    portion comes from ``state`` (float32 ``[slots + 1, taps - 1, channels]``: the request's last
    inputs, oldest first), which then receives the last inputs of this step."""
    tokens = proj.shape[0]
    taps, channels = weight.shape
    requests = slots.shape[0]
    _run("recurrence", "b200_causal_conv_silu",
         _P(_check("projection", proj, _RUN, (tokens, None))), _I(proj.shape[1]), _I(offset),
         _P(_check("conv weight", weight, torch.float32)), _P(_check("conv bias", bias, torch.float32, (channels,))),
         _P(_check("conv state", state, torch.float32, (None, taps - 1, channels))),
         _P(_check("request of each token", token_request, torch.int32, (tokens,))),
         _P(_check("query_start", query_start, torch.int32, (requests + 1,))),
         _P(_check("state slots", slots, torch.int32, (requests,))),
         _P(_check("convolved output", out, torch.float32, (tokens, channels))),
         _I(tokens), _I(requests), _I(channels), _I(taps), _I(_code(proj.dtype)), _stream())
    if taps > 1:
        count_launch()          # the kernel that replaces the state
