"""Python face of the kernels for differential attention: two softmax maps to a head over the same values,
the second subtracted from the first (``csrc/diff_attention.cu``).

As everywhere in this package there is no CPU or library alternative behind these functions.
"""

from __future__ import annotations

import torch

from ..csrc.build import load_library
from . import _F, _I, _P, KernelError, _check, _code, _run, _stream, count_launch

_RUN = (torch.float32, torch.bfloat16)
MAPS = 2
# bfloat16 batches go to the tensor-core kernels where their sizes allow (False: the float32 kernel for everything).
USE_TENSOR_CORES = True
SHARED_MEMORY_LIMIT = 220 * 1024


_sms: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _sms:
        _sms[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sms[index]


def tensor_core_sizes_ok(head_dim: int, value_dim: int) -> bool:
    """Whether ``csrc/diff_attention_bf16.cu`` can be compiled for these sizes: multiples of 16, the value head at
    most 256 (a thread's registers hold its part of an output row), and the decode kernel's three stages of a tile
    of 64 keys and values, as well as its room for its warps' partial results, within a block's shared memory."""
    if head_dim % 16 or value_dim % 16 or head_dim <= 0 or not 0 < value_dim <= 256:
        return False
    stages = 3 * 64 * ((MAPS * head_dim + 8) + (value_dim + 8)) * 2 + 3 * 64 * 8     # and where each entry's row lies
    merge = (8 * 16 * value_dim + 8 * 16 * 2 + 2 * 16 * value_dim) * 4
    return max(stages, merge) <= SHARED_MEMORY_LIMIT


def decode_splits(num_requests: int, num_kv_heads: int, keys: int, sms: int) -> int:
    """Over how many blocks the keys of one (request, key/value head) of a decode batch are split: at least 256
    keys to a block, at most 16 blocks, and so many that the blocks fill whole rounds of the GPU (two blocks to an
    SM at a time) as nearly as possible; a split more costs a little.  Pairs that fill the GPU by themselves are
    not split."""
    pairs = max(1, num_requests * num_kv_heads)
    slots = 2 * sms
    if pairs >= slots:
        return 1
    best, best_fill = 1, 0.0
    for splits in range(1, max(1, min(16, keys // 256)) + 1):
        blocks = pairs * splits
        fill = blocks / (-(-blocks // slots) * slots) - 0.002 * splits
        if fill > best_fill:
            best, best_fill = splits, fill
    return best


def bias_rope_cache(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor,
                    inv_freq: torch.Tensor | None, rotary_dim: int, q_out: torch.Tensor, k_pages: torch.Tensor | None,
                    v_pages: torch.Tensor | None, num_q_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                    page_size: int) -> None:
    """From the packed projection ``[T, (nq + nkv) * 2 d + nkv * dv]`` (every query and key head holds its two
    maps side by side): ``bias`` (float32, the same width) added, the first ``rotary_dim`` numbers of every map
    rotated by the token's position (pairs ``(i, i + rotary_dim / 2)``, angle ``position * inv_freq[i]`` in
    float32), queries to ``q_out`` ``[T, nq * 2 d]``, keys to ``k_pages`` ``[pages, nkv, page_size, 2 d]`` and values
    to ``v_pages`` ``[pages, nkv, page_size, dv]`` at ``slots`` (negative slot: not stored; pages None: nothing is)."""
    tokens = qkv.shape[0]
    dtype = qkv.dtype
    width = (num_q_heads + num_kv_heads) * MAPS * head_dim + num_kv_heads * value_dim
    _run("diff_attention", "b200_bias_rope_cache",
         _P(_check("qkv", qkv, _RUN, (tokens, width))),
         _P(_check("projection bias", bias, torch.float32, (width,), optional=True)),
         _P(_check("positions", positions, torch.int32, (tokens,))),
         _P(_check("slot mapping", slots, torch.int32, (tokens,))),
         _P(_check("inverse frequencies", inv_freq, torch.float32, (rotary_dim // 2,), optional=rotary_dim == 0)),
         _P(_check("q output", q_out, dtype, (tokens, num_q_heads * MAPS * head_dim))),
         _P(_check("key pages", k_pages, dtype, (None, num_kv_heads, page_size, MAPS * head_dim), optional=True)),
         _P(_check("value pages", v_pages, dtype, (None, num_kv_heads, page_size, value_dim), optional=True)),
         _I(tokens), _I(num_q_heads * MAPS), _I(num_kv_heads), _I(MAPS), _I(head_dim), _I(value_dim), _I(rotary_dim),
         _I(page_size), _I(_code(dtype)), _stream())


def diff_paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                         query_start: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                         num_q_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, page_size: int,
                         scale: float, softcap: float | None, window: int | None, keep_first: int, lam: float,
                         eps: float, out_scale: float, max_query_len: int | None = None,
                         max_seq_len: int | None = None, num_decode: int = 0) -> None:
    """Differential attention of every request's new queries over its pages: per head ``o = a1 - lam * a2``
    with ``a_m = softmax_j(cap(q_m . k_mj * scale)) v_j`` over the keys ``j <= i`` with ``i - j < window`` or ``j <
    keep_first``, ``cap(s) = softcap * tanh(s / softcap)``; then ``out = o * rsqrt(mean(o^2) + eps) * out_scale``
    over the head's ``dv`` values.  Scores, weights, sums and the norm in float32."""
    tokens = q.shape[0]
    requests = seq_lens.shape[0]
    dtype = q.dtype
    checked = (
        _check("queries", q, _RUN, (tokens, num_q_heads * MAPS * head_dim)),
        _check("key pages", k_pages, dtype, (None, num_kv_heads, page_size, MAPS * head_dim)),
        _check("value pages", v_pages, dtype, (None, num_kv_heads, page_size, value_dim)),
        _check("attention output", out, dtype, (tokens, num_q_heads * value_dim)),
        _check("query_start", query_start, torch.int32, (requests + 1,)),
        _check("seq_lens", seq_lens, torch.int32, (requests,)),
        _check("block table", block_table, torch.int32, (requests, None)))
    if keep_first < 0:
        raise KernelError(f"keep_first={keep_first}")
    if USE_TENSOR_CORES and dtype == torch.bfloat16 and tensor_core_sizes_ok(head_dim, value_dim):
        # The tensor-core kernels, compiled for this pair of sizes: one-token requests at the head of the batch
        # with their keys split over several blocks, portions of prompts in tiles of 64 queries.
        # one-token requests: all of a decode step, the first ``num_decode`` of a step that mixes them with prompts
        decode = requests if max_query_len == 1 and tokens == requests else num_decode
        if num_q_heads // num_kv_heads > 16:
            decode = 0
        splits, partial_o, partial_ml = 1, None, None
        if decode:
            keys = max_seq_len if max_seq_len is not None else block_table.shape[1] * page_size
            if window:
                keys = min(keys, window + keep_first)
            splits = decode_splits(decode, num_kv_heads, keys, _sm_count(q.device))
            if splits > 1:
                rows = decode * num_q_heads * MAPS * splits
                partial_o = torch.empty((rows, value_dim), dtype=torch.float32, device=q.device)
                partial_ml = torch.empty((rows, 2), dtype=torch.float32, device=q.device)
        lib = load_library("diff_attention_bf16", (("B200_DIFF_D", head_dim), ("B200_DIFF_DV", value_dim)))
        count_launch()
        status = lib.b200_diff_attention_bf16(
            *(_P(address) for address in checked), _I(requests), _I(tokens), _I(block_table.shape[1]),
            _I(num_q_heads), _I(num_kv_heads), _I(page_size), _F(scale), _F(softcap or 0.0), _I(window or 0),
            _I(keep_first), _F(lam), _F(eps), _F(out_scale), _I(decode), _I(splits),
            _P(partial_o.data_ptr() if partial_o is not None else 0),
            _P(partial_ml.data_ptr() if partial_ml is not None else 0), _stream())
        if status != 0:
            raise KernelError(lib.b200_last_error().decode())
        return
    _run("diff_attention", "b200_diff_paged_attention", *(_P(address) for address in checked),
         _I(requests), _I(tokens), _I(block_table.shape[1]), _I(num_q_heads), _I(num_kv_heads), _I(head_dim),
         _I(value_dim), _I(page_size), _F(scale), _F(softcap or 0.0), _I(window or 0), _I(keep_first), _F(lam), _F(eps),
         _F(out_scale), _I(_code(dtype)), _stream())
