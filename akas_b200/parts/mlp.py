"""A dense feed-forward without a gate: W_down act(W_up x).

``activation``: "relu2" (the square of max(z, 0)), "gelu_tanh" or "silu". The activation is float32, computed on the
up product's float32 sums (in the product's read-out where the kernels offer ``ops.linear_activated``, else by
``ops.activation`` on a float32 product) and rounded once to the compute dtype as the down product's operand.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Normed, Param, project, register_ffn, renamed

ACTIVATIONS = ("relu2", "gelu_tanh", "silu")


def project_activated(rt, x, w_up, activation):
    """``act(x . w_up^T)`` in the compute dtype, for a tensor or a ``Normed``."""
    ops = rt.ops
    if isinstance(x, Normed):
        if getattr(x.norm.spec, "kind", None) == "dynamic_tanh" and hasattr(ops, "dyt_linear_activated"):
            out = ops.dyt_linear_activated(x.h, x.norm.alpha, x.norm.weight, x.norm.shift, w_up, activation, x.rows)
            if out is not None:
                return out
        x = x.tensor()
    if hasattr(ops, "linear_activated"):
        out = ops.linear_activated(x, w_up, activation)
        if out is not None:
            return out
    return ops.activation(ops.linear(x, w_up, out_dtype=torch.float32), activation, rt.dtype)


class MLP(FeedForward):
    takes_normed = True
    chain_safe = True
    takes_out_dtype = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {list(ACTIVATIONS)}")
        self.w_up = self.w_down = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        c, f = self.spec.hidden_size, self.spec.intermediate_size
        return {self._n("up"): Param((f, c)), self._n("down"): Param((c, f))}

    def load(self, get):
        self.w_up, self.w_down = get(self._n("up")), get(self._n("down"))

    def forward(self, x, ctx, residual=None, out_dtype=None):
        act = project_activated(self.rt, x, self.w_up, self.spec.activation)
        return project(self.rt, act, self.w_down, out_dtype=out_dtype, residual=residual)


register_ffn("mlp", MLP)
