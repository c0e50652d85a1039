"""A routed feed-forward: a mixture of SwiGLU experts, a few per token, some of them identities.

Per token (all of the router in float32): scores = softmax(W_router x) over every router output; the choice goes by
score + correction among the outputs of the best groups of neighbours; the weights are the chosen outputs' plain
scores over their sum; the result is the weighted sum of the chosen experts' W_down (silu(W_gate x) * (W_up x)),
where a router output past the real experts stands for an expert that returns x. The experts' matrices are stacked
at load ([experts, 2 F, C] with the gate rows first, and [experts, C, F]), so the kernels address an expert by its
number.

Options of the spec change the rule: sigmoid scores instead of a softmax, no correction, weights that are the chosen
scores as they are, a weight that multiplies the expert's input (sum expert(w x)) instead of its result, and one more
expert that every token passes, whose result is added to the sum, times sigmoid(W_sg x) (one number per token) where
the spec says so. That expert is a gated feed-forward on the products' own kernels; its gate's logit is one more row
of the router's float32 matrix, and the experts' last kernel adds its result to theirs.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Param, project, project_gated, register_ffn, renamed, stack_rows


class RoutedExperts(FeedForward):
    chain_safe = True
    takes_out_dtype = True

    @classmethod
    def kernels(cls, spec):
        return ("moe",)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        outputs = s.num_experts + s.num_identity
        if s.num_experts < 1 or s.num_identity < 0:
            raise ValueError("a mixture needs at least one real expert")
        if s.groups < 1 or outputs % s.groups or not 1 <= s.keep_groups <= s.groups:
            raise ValueError(f"{outputs} router outputs do not form {s.groups} equal groups of which {s.keep_groups} stay")
        if not 1 <= s.top <= s.keep_groups * (outputs // s.groups):
            raise ValueError(f"top {s.top} exceeds what {s.keep_groups} groups of {outputs // s.groups} offer")
        self.scoring = getattr(s, "scoring", "softmax")
        self.weight_input = getattr(s, "weight_on", "output") == "input"
        if self.scoring not in ("softmax", "sigmoid") or getattr(s, "weight_on", "output") not in ("output", "input"):
            raise ValueError(f"unknown scoring {self.scoring!r} or weight_on {s.weight_on!r}")
        if self.weight_input and s.num_identity:
            raise ValueError("a weight on the expert's input leaves identity experts without a rule")
        self.shared_size = getattr(s, "shared_size", None)
        self.shared_gate = bool(getattr(s, "shared_gate", False)) and self.shared_size is not None
        self.has_correction = bool(getattr(s, "correction", True))
        self.renormalize = bool(getattr(s, "renormalize", True))
        # the plain rule keeps the call it always made; anything else names its options
        self.plain_rule = (self.scoring == "softmax" and self.has_correction and self.renormalize and not self.weight_input
                           and self.shared_size is None)
        self.w_router = self.correction = self.w_gate_up = self.w_down = None
        self.w_shared_gate_up = self.w_shared_down = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        c, f, outputs = s.hidden_size, s.intermediate_size, s.num_experts + s.num_identity
        p = {self._n("router"): Param((outputs, c), role="vector")}  # held in float32: the router's own precision
        if self.has_correction:
            p[self._n("correction")] = Param((outputs,), role="vector")
        if self.shared_size is not None:
            fs = self.shared_size
            p[self._n("shared.gate")] = Param((fs, c))
            p[self._n("shared.up")] = Param((fs, c))
            p[self._n("shared.down")] = Param((c, fs))
            if self.shared_gate:
                p[self._n("shared.sg")] = Param((1, c), role="vector")
        for e in range(s.num_experts):
            p[self._n(f"e{e}.gate")] = Param((f, c))
            p[self._n(f"e{e}.up")] = Param((f, c))
            p[self._n(f"e{e}.down")] = Param((c, f))
        return p

    def load(self, get):
        s = self.spec
        self.w_router = get(self._n("router"))
        self.correction = get(self._n("correction")) if self.has_correction else None
        if self.shared_size is not None:
            self.w_shared_gate_up = stack_rows([get(self._n("shared.gate")), get(self._n("shared.up"))])
            self.w_shared_down = get(self._n("shared.down"))
            if self.shared_gate:  # the gate's logit is one more output of the router's product
                self.w_router = torch.cat([self.w_router, get(self._n("shared.sg")).reshape(1, -1)], dim=0).contiguous()
        self.w_gate_up = torch.stack(
            [torch.cat([get(self._n(f"e{e}.gate")), get(self._n(f"e{e}.up"))], dim=0) for e in range(s.num_experts)]
        ).contiguous()
        self.w_down = torch.stack([get(self._n(f"e{e}.down")) for e in range(s.num_experts)]).contiguous()

    def _route(self, x):
        """(chosen, weights, the shared expert's gate [N, 1] or None)."""
        s, ops = self.spec, self.rt.ops
        if self.plain_rule:
            return (*ops.moe_route(x, self.w_router, self.correction, s.groups, s.keep_groups, s.top), None)
        routed = ops.moe_route(x, self.w_router, self.correction, s.groups, s.keep_groups, s.top, scoring=self.scoring,
                               renormalize=self.renormalize, extra=int(self.shared_gate))
        return routed if self.shared_gate else (*routed, None)

    def _experts(self, x, update=None):
        ops = self.rt.ops
        chosen, weights, gate = self._route(x)
        more = {}
        if self.weight_input:
            more["weight_input"] = True
        if self.shared_size is not None:
            # the expert that every token passes: a gated feed-forward on the products' kernels, float32 out; the
            # experts' last kernel adds it, times its gate
            act = project_gated(self.rt, x, self.w_shared_gate_up, self.shared_size, None, "silu")
            more["shared"] = (project(self.rt, act, self.w_shared_down, out_dtype=torch.float32), gate)
        return ops.moe_experts(x, self.w_gate_up, self.w_down, chosen, weights, update=update, **more)

    def forward_update(self, x, ctx, h, a, scale_a, scale_b, mult):
        """h += mult * (scale_a * a + scale_b * experts(x)) in place on the float32 residual stream h, by the experts' last
        kernel: what a block whose sublayers' results meet the stream in one sum asks for."""
        return self._experts(x, update=(h, a, scale_a, scale_b, mult))

    def forward(self, x, ctx, residual=None, out_dtype=None):
        ops = self.rt.ops
        out = self._experts(x)  # float32 [N, C]
        if residual is not None:
            return ops.scaled_add(residual, out, None, None, None, 1.0)
        return out if out_dtype in (None, torch.float32) else out.to(out_dtype)


register_ffn("routed_experts", RoutedExperts)
