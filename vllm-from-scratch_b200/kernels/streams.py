"""Python face of the kernel for a residual that is kept as several streams (``csrc/streams.cu``).

As everywhere in this package there is no CPU or library alternative behind these functions.
"""

from __future__ import annotations

import torch

from . import _F, _I, _P, KernelError, _check, _code, _run, _stream

_RUN = (torch.float32, torch.bfloat16)
MAX_STREAMS = 16


def stream_mix_norm(streams: torch.Tensor, *, rows_in: torch.Tensor | None = None, mix: torch.Tensor | None = None,
                    out_weights: torch.Tensor | None = None, fresh: torch.Tensor | None = None,
                    in_weights: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None, eps: float = 0.0,
                    normed: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> None:
    """What lies between two sublayers of a model whose residual is ``streams`` (float32 ``[T, S, H]``), as one
    kernel, every part optional:

    * the update by the sublayer behind, ``X'_t = sum_s mix[s, t] X_s + out_weights[t] rows_in`` (``rows_in``
      ``[T, H]`` in the run dtype, ``mix`` float32 ``[S, S]`` indexed ``[from, to]``), in place; or ``fresh``
      (float32 ``[T, H]``): every stream is set to it;
    * the read by the sublayer ahead, ``u = sum_t in_weights[t] X'_t`` (``in_weights`` None: the plain sum), and
      its RMSNorm ``normed = u * rsqrt(mean(u^2) + eps) * norm_weight`` (``normed`` None: the update only).

    With ``rows`` (int32 row numbers) only those rows are read and normalised, written one after another to
    ``normed``, and ``streams`` stays as it was."""
    tokens, count, hidden = streams.shape
    if count > MAX_STREAMS:
        raise KernelError(f"{count} streams: up to {MAX_STREAMS} are built")
    out_rows = tokens if rows is None else rows.shape[0]
    if normed is None and rows is not None:
        raise KernelError("stream_mix_norm: a list of rows without an output does nothing")
    dtype = normed.dtype if normed is not None else rows_in.dtype if rows_in is not None else torch.float32
    _run("streams", "b200_stream_mix_norm",
         _P(_check("rows on their way into the streams", rows_in, dtype, (tokens, hidden), optional=True)),
         _P(_check("fresh rows", fresh, torch.float32, (tokens, hidden), optional=True)),
         _P(_check("stream mix", mix, torch.float32, (count, count), optional=True)),
         _P(_check("stream out weights", out_weights, torch.float32, (count,), optional=True)),
         _P(_check("streams", streams, torch.float32)),
         _P(_check("stream in weights", in_weights, torch.float32, (count,), optional=True)),
         _P(_check("norm weight", norm_weight, torch.float32, (hidden,), optional=True)), _F(eps),
         _P(_check("norm output", normed, _RUN, (out_rows, hidden), optional=True)),
         _P(_check("row index", rows, torch.int32, optional=True)),
         _I(out_rows), _I(count), _I(hidden), _I(_code(dtype)), _stream())
