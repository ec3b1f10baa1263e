"""Partial rotary position encoding with optional sections.

``inv_freq[j] = theta ** (-2j / rotary_dim)`` for the ``rotary_dim / 2`` rotate-half pairs ``(j, j +
rotary_dim/2)`` of the first ``rotary_dim`` dims of a head; the rest of the head is not rotated
(src/quanta/minimax/model_m3.py:68-96).  With ``sections`` the pairs are split into runs, run ``a``
taking position axis ``a`` (src/quanta/minimax/model_vision_m3.py:155-163); a text token feeds its
one position to every axis, so the numbers equal the unsectioned ladder.

``wavelength_scaling = (factor, low, high, original)`` rescales the ladder by wavelength ``l = 2 pi / f``: a
frequency whose wavelength is shorter than ``original / high`` is kept, one longer than ``original / low`` is
divided by ``factor``, and between the two, with ``s = (original / l - low) / (high - low)``, it becomes
``(1 - s) f / factor + s f``.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register


@register("position", "partial_rotary")
class PartialRotary(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, sections=None, wavelength_scaling=None):
        if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        if sections is not None and sum(sections) != rotary_dim // 2:
            raise ValueError(f"rope sections {list(sections)} do not sum to rotary_dim/2 = {rotary_dim // 2}")
        self.head_dim, self.rotary_dim, self.theta = int(head_dim), int(rotary_dim), float(theta)
        self.sections = None if sections is None else tuple(int(s) for s in sections)
        self.n_axes = 1 if self.sections is None else len(self.sections)
        self.wavelength_scaling = None
        if wavelength_scaling is not None:
            factor, low, high, original = (float(v) for v in wavelength_scaling)
            if factor <= 0 or original <= 0 or low <= 0 or high <= low:
                raise ValueError(f"wavelength scaling {tuple(wavelength_scaling)}: needs factor, original > 0 and "
                                 f"0 < low < high")
            self.wavelength_scaling = (factor, low, high, original)
        self._tables = {}

    def inv_freq(self) -> torch.Tensor:
        rd = self.rotary_dim
        if self.wavelength_scaling is None:
            return 1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        # the ladder and its rescaling in float64, rounded once to the float32 the kernels multiply positions with
        f = self.theta ** (-torch.arange(0, rd, 2, dtype=torch.float64) / rd)
        factor, low, high, original = self.wavelength_scaling
        wavelength = 2.0 * math.pi / f
        s = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
        blended = (1.0 - s) * f / factor + s * f
        out = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
        return out.to(torch.float32)

    def rotary_tables(self, device):
        if self.rotary_dim == 0:
            return None
        key = str(device)
        if key not in self._tables:
            inv = self.inv_freq().to(device)
            axis = None
            if self.sections is not None:
                axis = torch.cat([torch.full((n,), a, dtype=torch.int32) for a, n in enumerate(self.sections)])
                axis = axis.to(device)
            self._tables[key] = (inv, axis, self.rotary_dim, self.n_axes)
        return self._tables[key]


@register("position", "none")
class NoPosition(PositionEncoding):
    """Nothing is rotated: positions reach the mixer some other way (a learned table, a query temperature)."""

    graph_safe = True

    def rotary_tables(self, device):
        return None
