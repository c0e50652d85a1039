"""A gated feed-forward with a choice of activation and optional biases:
W_down (act(W_gate x + b_gate) * (W_up x + b_up)) + b_down.

W_gate and W_up are stacked at load so that one product feeds the activation. The biases, the activation and the
product of the two halves are float32, computed on the product's float32 sums in its read-out (``ops.linear_gated``;
where the kernels do not offer that, the product leaves float32 and ``ops.gated_activation`` follows) and rounded once
to the compute dtype as the down product's operand. The down product adds its sums and its bias into the float32
residual stream.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Param, project, project_gated, register_ffn, renamed, stack_rows

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
        act = project_gated(self.rt, x, self.w_gate_up, self.spec.intermediate_size, self.bias_gate_up, self.spec.activation)
        if residual is None:
            out = project(self.rt, act, self.w_down, out_dtype=torch.float32, bias=self.bias_down)
            return out.to(self.rt.dtype)
        return project(self.rt, act, self.w_down, residual=residual, bias=self.bias_down)


register_ffn("gated_mlp", GatedMLP)
