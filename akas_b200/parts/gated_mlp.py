"""A gated feed-forward with a choice of activation and optional biases:
W_down (act(W_gate x + b_gate) * (W_up x + b_up)) + b_down.

W_gate and W_up are stacked at load so that one product feeds the activation. That product leaves float32; the
biases, the activation and the product of the two halves are float32 (``ops.gated_activation``), rounded once to the
compute dtype as the down product's operand. The down bias is added to the float32 residual stream by the
activation's launch; the down product then accumulates into that stream.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Param, project, register_ffn, renamed, stack_rows

ACTIVATIONS = ("gelu_tanh", "silu")


class GatedMLP(FeedForward):
    takes_normed = True
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {list(ACTIVATIONS)}")
        self.w_gate_up = self.w_down = self.bias_gate_up = self.bias_down = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        c, f = self.spec.hidden_size, self.spec.intermediate_size
        p = {self._n("gate"): Param((f, c)), self._n("up"): Param((f, c)), self._n("down"): Param((c, f))}
        if self.spec.bias:
            p[self._n("gate") + ".b"] = Param((f,), role="vector")
            p[self._n("up") + ".b"] = Param((f,), role="vector")
            p[self._n("down") + ".b"] = Param((c,), role="vector")
        return p

    def load(self, get):
        self.w_gate_up = stack_rows([get(self._n("gate")), get(self._n("up"))])
        self.w_down = get(self._n("down"))
        if self.spec.bias:
            self.bias_gate_up = torch.cat([get(self._n("gate") + ".b"), get(self._n("up") + ".b")]).contiguous()
            self.bias_down = get(self._n("down") + ".b")

    def forward(self, x, ctx, residual=None):
        ops = self.rt.ops
        gate_up = project(self.rt, x, self.w_gate_up, out_dtype=torch.float32)
        more = {}
        if residual is not None and self.bias_down is not None:
            more = dict(residual=residual, residual_bias=self.bias_down)  # the same launch adds the last product's bias
        act = ops.gated_activation(gate_up, self.spec.intermediate_size, self.bias_gate_up, self.spec.activation, self.rt.dtype,
                                   **more)
        if residual is None:
            out = project(self.rt, act, self.w_down, out_dtype=torch.float32)
            return ops.add_bias(out, self.bias_down, self.rt.dtype) if self.bias_down is not None else out.to(self.rt.dtype)
        return project(self.rt, act, self.w_down, residual=residual)


register_ffn("gated_mlp", GatedMLP)
