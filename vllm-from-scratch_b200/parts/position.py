"""Position encodings of the rotary family.

``rotary``: rotate-half ("neox") rotation of the first ``rotary_dim`` channels of
every query and key head by the angle ``position * theta^(-2j / rotary_dim)``
(minivllm/layers/rotary_embedding.py:143-185 builds the same frequencies;
minivllm/layers/ops/rotary_embedding.py:243-257 applies them).  The reference
tabulates cos/sin per position and casts the table to the run dtype; here the
angle is formed and its sine and cosine taken in float32 inside the kernel, so
only the frequencies are stored.

With ``frequency_scaling = (factor, low, high, original)`` the frequencies of long wavelengths are
lowered: a frequency f whose wavelength ``l = 2 pi / f`` is below ``original / high`` stays, one whose
wavelength is above ``original / low`` becomes ``f / factor``, and between the two, with ``s = (original / l
- low) / (high - low)``, it becomes ``(1 - s) f / factor + s f``.

``none``: no rotation.
"""

from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from .base import POSITION_ENCODINGS, PartEnv, PositionEncoding


@POSITION_ENCODINGS.register("rotary")
class RotaryPositionEncoding(PositionEncoding):
    """params: ``theta`` (base), ``rotary_dim`` (channels rotated, even),
    ``scaling_factor`` (positions are divided by it; 1.0 = plain), ``frequency_scaling`` (``(factor, low,
    high, original)`` or None: the stretching of long wavelengths described above), ``interleaved`` (default
    False: channel i is turned with channel ``i + rotary_dim / 2``; True: channel 2i with channel 2i + 1.  A mixer's
    kernel must know the second form; the frequencies are formed in double precision and rounded once with it)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        self.scaling_factor = float(params.get("scaling_factor", 1.0))
        self.interleaved = bool(params.get("interleaved", False))
        if self.theta <= 0 or self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary position encoding: theta={self.theta}, rotary_dim={self.rotary_dim}")
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponents)
        if self.scaling_factor != 1.0:
            inv_freq = inv_freq / self.scaling_factor
        scaling = params.get("frequency_scaling")
        self.frequency_scaling = None if scaling is None else tuple(float(v) for v in scaling)
        if self.frequency_scaling is not None:
            factor, low, high, original = self.frequency_scaling
            if factor <= 0 or low <= 0 or high <= low or original <= 0:
                raise ValueError(f"rotary position encoding: frequency_scaling={self.frequency_scaling}")
            made = []
            for pair in range(self.rotary_dim // 2):        # in double precision, rounded once at the end
                f = self.theta ** (-2.0 * pair / self.rotary_dim) / self.scaling_factor
                wavelength = 2.0 * math.pi / f
                if wavelength > original / low:
                    f = f / factor
                elif wavelength >= original / high:
                    smooth = (original / wavelength - low) / (high - low)
                    f = (1.0 - smooth) * f / factor + smooth * f
                made.append(f)
            inv_freq = torch.tensor(made, dtype=torch.float64).to(torch.float32)
        elif self.interleaved:
            made = [self.theta ** (-2.0 * pair / self.rotary_dim) / self.scaling_factor for pair in range(self.rotary_dim // 2)]
            inv_freq = torch.tensor(made, dtype=torch.float64).to(torch.float32)
        self._inv_freq = inv_freq.to(env.device)

    def inverse_frequencies(self) -> torch.Tensor:
        return self._inv_freq


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    rotary_dim = 0
    graph_safe = True
