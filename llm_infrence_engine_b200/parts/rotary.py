"""Rotary position encoding: per-step cosine and sine tables from the tokens' absolute positions."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """Angles ``position * theta^(-2j/d)`` for ``j < d/2``, in 32-bit; pairs are ``(j, j + d/2)``.

    The inverse frequencies are made the way the reference makes them (32-bit power and division,
    src/miniserve/model.py:83-85) so that both sides round alike; the reference then recomputes
    ``cos`` and ``sin`` on every forward (model.py:86-88), here the step does it once for all layers.
    """

    graph_safe = True

    def __init__(self, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError(f"rotary head_dim must be even, got {head_dim}")
        self.head_dim = head_dim
        self.theta = float(theta)
        self._inv_freq = {}

    def key(self) -> tuple:
        return ("rotary", self.head_dim, self.theta)

    def inv_freq(self, device) -> torch.Tensor:
        dev = str(device)
        if dev not in self._inv_freq:
            f = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2).float() / self.head_dim))
            self._inv_freq[dev] = f.to(device)
        return self._inv_freq[dev]

    def tables(self, ctx):
        """(cos, sin), each ``[N, head_dim / 2]`` in 32-bit."""
        return ctx.K.rope_tables(ctx.positions, self.inv_freq(ctx.device))


class RampedRotary(PositionEncoding):
    """Rotation angles ``position * f_i`` for ``i < dims / 2`` whose frequencies are stretched by wavelength (the scheme known
    as YaRN): with ``f_i = base^(-2i/dims)``, ``d(t) = dims ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(d(fast)), 0)``,
    ``hi = min(ceil(d(slow)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency is
    ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and cos and sin are both multiplied by ``0.1 ln(factor) + 1``. Without
    ``factor`` the frequencies are plain. The frequencies are made once, in 64-bit, and rounded to 32-bit; the angles are
    32-bit products. Which entries of a head form a pair is the mixer's business, not the table's.
    """

    graph_safe = True

    def __init__(self, dims: int, base: float, factor: Optional[float] = None, original: float = 0.0, fast: float = 32.0, slow: float = 1.0):
        if dims <= 0 or dims % 2:
            raise ValueError(f"the rotated dimensions must be even and positive, got {dims}")
        self.dims, self.base = int(dims), float(base)
        self.factor = None if factor is None else float(factor)
        self.original, self.fast, self.slow = float(original), float(fast), float(slow)
        self._inv_freq = {}

    def key(self) -> tuple:
        return ("ramped-rotary", self.dims, self.base, self.factor, self.original, self.fast, self.slow)

    def frequencies(self) -> list:
        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        if self.factor is None:
            return f

        def dim_of(turns: float) -> float:
            return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo = max(math.floor(dim_of(self.fast)), 0)
        hi = min(math.ceil(dim_of(self.slow)), self.dims - 1)
        out = []
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f[i] / self.factor * ramp + f[i] * (1.0 - ramp))
        return out

    @property
    def magnitude(self) -> float:
        return 1.0 if self.factor is None else 0.1 * math.log(self.factor) + 1.0

    def inv_freq(self, device) -> torch.Tensor:
        dev = str(device)
        if dev not in self._inv_freq:
            self._inv_freq[dev] = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32).to(device)
        return self._inv_freq[dev]

    def tables(self, ctx):
        """(cos, sin), each ``[N, dims / 2]`` in 32-bit, the magnitude already on them."""
        return ctx.K.rope_tables(ctx.positions, self.inv_freq(ctx.device), self.magnitude)
