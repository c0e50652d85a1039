"""Norms. RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w. Dynamic Tanh: y = tanh(alpha * x) * w + b. Both in float32.

kreasof-ai/akas: src/akas/ops/normalization/kernel.py:440-444; the weight is used
as it stands (its ``zero_centered`` flag, 1 + w, belongs to other contracts:
src/akas/ops/normalization/definition.py:285-348) and is offered here as an option.
"""

from __future__ import annotations

import torch

from .base import Normed, Param, Part, register_norm


class RMSNorm(Part):
    chain_safe = True

    def __init__(self, spec, runtime, name: str = "weight"):
        super().__init__(spec, runtime)
        self.name = name
        self.weight = None

    def params(self):
        return {self.name: Param((self.spec.size,), role="vector", mean=0.0 if self.spec.zero_centered else 1.0)}

    def load(self, get):
        self.weight = get(self.name)

    def forward(self, x, out_dtype=None, rows=None):
        """x: [N, size] (or [N, heads, size] flattened by the caller); rows: optional int32 row indices."""
        return self.rt.ops.rmsnorm(
            x, self.weight, self.spec.eps, self.spec.zero_centered, out_dtype or self.rt.dtype, rows
        )


    def lazy(self, h, rows=None) -> Normed:
        return Normed(self, h, rows)


class DynamicTanh(Part):
    """tanh(alpha * x) * w + b, element by element: a norm without a mean or a variance, so a token's row needs no
    sum. alpha is one learned number (kept on the device: nothing waits for it), w and b vectors of the row's size.
    Its tensors: the weight, and beside it ``.alpha`` and ``.b``."""

    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.weight = self.alpha = self.shift = None

    def params(self):
        n = self.spec.size
        return {"weight": Param((n,), role="vector", mean=1.0), ".alpha": Param((), role="vector", mean=0.5),
                ".b": Param((n,), role="vector")}

    def load(self, get):
        self.weight, self.alpha, self.shift = get("weight"), get(".alpha"), get(".b")

    def forward(self, x, out_dtype=None, rows=None):
        """x: float32 [N, size]; rows: optional int32 row indices (only those rows are normed and returned)."""
        return self.rt.ops.dynamic_tanh(x, self.alpha, self.weight, self.shift, out_dtype or self.rt.dtype, rows)

    def lazy(self, h, rows=None) -> Normed:
        return Normed(self, h, rows)

    def add_to(self, y, h):
        """h += norm(y) in place on the float32 stream h [N, size], for float32 y: the norm behind a sublayer and the
        residual sum as one kernel."""
        return self.rt.ops.dynamic_tanh(y, self.alpha, self.weight, self.shift, torch.float32, residual=h)


register_norm("rmsnorm", RMSNorm)
register_norm("dynamic_tanh", DynamicTanh)
