"""Rotary position encoding, rotate-half pairing (i, i + rotary/2) or interleaved pairing (2i, 2i + 1).

theta_i = position * base^(-2i/rotary). kreasof-ai/akas forms this product with a
hi/lo split of the frequency and a two-term reduction by 2 pi so that float32 stays
accurate at long positions (src/akas/ops/attention/kernel.py:788-851, 927-939). Here
the frequencies are float64 constants made once on the host, and the kernel
multiplies, reduces and rounds to float32 last; the tables of a step are made once
and shared by every layer with the same encoding.
"""

from __future__ import annotations

import math

import torch

from .base import Part, register_position


def slow_long_waves(freq: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """The rates of rotary pairs with long waves slowed (float64, on the host): with wavelength l = 2 pi / f a pair keeps
    f where l < original / high, gets f / factor where l > original / low, and in between
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    wave = 2.0 * math.pi / freq
    s = (original / wave - low) / (high - low)
    blended = (1.0 - s) * freq / factor + s * freq
    return torch.where(wave > original / low, freq / factor, torch.where(wave < original / high, freq, blended))


def blend_by_index(freq: torch.Tensor, theta: float, rotary: int, factor: float, original: float, fast: float,
                   slow: float) -> torch.Tensor:
    """The rates of rotary pairs blended by the pair's index (float64, on the host): with
    d(t) = rotary ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary - 1)
    and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at r_i f_i / factor + (1 - r_i) f_i: the pairs
    below lo keep their rate, those above hi turn ``factor`` times slower."""

    def d(turns: float) -> float:
        return rotary * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo, hi = max(math.floor(d(fast)), 0), min(math.ceil(d(slow)), rotary - 1)
    i = torch.arange(freq.numel(), dtype=torch.float64)
    r = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * r + freq * (1.0 - r)


class Rope(Part):
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        rotary = spec.rotary
        if rotary % 2 or rotary > spec.head_dim or rotary <= 0:
            raise ValueError(f"rotary_dim {rotary} must be even and at most head_dim {spec.head_dim}")
        i = torch.arange(rotary // 2, dtype=torch.float64)
        freq = torch.tensor(float(spec.theta), dtype=torch.float64) ** (-2.0 * i / rotary)
        scaling = getattr(spec, "scaling", None)
        if scaling is not None:
            freq = slow_long_waves(freq, *scaling)
        linear, blend = getattr(spec, "linear_factor", None), getattr(spec, "blend", None)
        if linear is not None:
            freq = freq / float(linear)
        if blend is not None:
            freq = blend_by_index(freq, float(spec.theta), rotary, *blend)
        self.amplitude = float(getattr(spec, "amplitude", 1.0))
        self.inv_freq = freq.to(runtime.device)
        # the tables are the same for both pairings
        self.key = ("rope", rotary, float(spec.theta), scaling, linear, blend, self.amplitude)
        self.interleaved = bool(getattr(spec, "interleaved", False))

    def tables(self, ctx):
        """(cos, sin), float32 [N, rotary/2], for the tokens of this step."""
        cached = ctx.memo.get(self.key)
        if cached is None:
            if self.amplitude != 1.0:
                cached = self.rt.ops.rope_tables(ctx.positions, self.inv_freq, self.amplitude)
            else:
                cached = self.rt.ops.rope_tables(ctx.positions, self.inv_freq)
            ctx.memo[self.key] = cached
        return cached


register_position("rope", Rope)
