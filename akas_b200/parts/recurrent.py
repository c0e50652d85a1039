"""Mixers whose cache is a matrix state per head: gated linear attention, linear attention with a constant decay per
head, and the gated delta rule.

All keep, per request and head, a float32 matrix S [key_dim, value_dim] in the request's state slot, update it
token by token and read it out with the token's query, so a step of any length continues from what earlier
steps left and a request's cost per token does not grow with its length.

* ``GatedLinearAttention``: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with a decay per key channel
  alpha = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau). (Yang et al., "Gated Linear Attention Transformers with
  Hardware-Efficient Training", state the recurrence.)
* ``DecayedLinearAttention``: S <- decay_h S + k_t v_t^T, o_t = S^T q_t with one constant decay per head (the
  recurrence of Qin et al.'s "Lightning Attention-2" without its chunking); q, k and v pass silu, the read-out of all
  heads is normed as one row, gated by sigmoid(W_g x) and projected.
* ``GatedDelta``: S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t, after a short causal
  convolution and silu on q, k and v and unit-length q and k. The convolution's last inputs are part of the state.

One product feeds everything that reads the mixer's input (the matrices are stacked at load); the decays, gates,
unit norms, the recurrence and the norm of its output are float32 whatever the compute dtype.
"""

from __future__ import annotations

import torch

from .base import Mixer, Param, StateSpec, project, register_mixer, renamed, stack_rows


class GatedLinearAttention(Mixer):
    takes_normed = True
    chain_safe = True

    @classmethod
    def kernels(cls, spec):
        return ("recurrent",)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.w_in = self.w_out = self.w_up = self.b_up = self.norm = None
        self.rank = spec.decay_rank

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        c, hd, hv = s.hidden_size, s.num_heads * s.key_dim, s.num_heads * s.value_dim
        rank = -1 if s.decay_rank is None else s.decay_rank
        default = max(8, s.key_dim // 2)
        return {
            self._n("q"): Param((hd, c)),
            self._n("k"): Param((hd, c)),
            self._n("v"): Param((hv, c)),
            self._n("g"): Param((hv, c)),
            self._n("o"): Param((c, hv)),
            self._n("norm"): Param((s.value_dim,), role="vector", mean=1.0),
            self._n("a1"): Param((rank, c), default=(default, c)),
            self._n("a2"): Param((hd, rank), role="vector", default=(hd, default)),
            self._n("a2.b"): Param((hd,), role="vector", mean=2.0),
        }

    def load(self, get):
        a1, up = get(self._n("a1")), get(self._n("a2"))
        self.rank = a1.shape[0]
        if up.shape[1] != self.rank:
            raise ValueError(f"the decay's two matrices disagree on their rank: {a1.shape[0]} and {up.shape[1]}")
        self.w_up = up.t().contiguous()  # [rank, heads * key_dim]: the gates' kernel reads it along its rows
        self.w_in = stack_rows([get(self._n("q")), get(self._n("k")), get(self._n("v")), get(self._n("g")), a1])
        self.b_up = get(self._n("a2.b"))
        self.norm = get(self._n("norm"))
        self.w_out = get(self._n("o"))

    def cache(self):
        s = self.spec
        return StateSpec((s.num_heads, s.value_dim, s.key_dim), torch.float32)  # S transposed, as the scan kernels keep it

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        s, ops = self.spec, self.rt.ops
        hd, hv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        proj = project(self.rt, x, self.w_in)
        q, k, v = proj[:, :hd], proj[:, hd : 2 * hd], proj[:, 2 * hd : 2 * hd + hv]
        gate = proj[:, 2 * hd + hv : 2 * hd + 2 * hv]
        low = proj[:, 2 * hd + 2 * hv : 2 * hd + 2 * hv + self.rank]
        alpha = ops.decay_gates(low, self.w_up, self.b_up, s.tau)
        o = ops.gla_scan(q, k, v, alpha, cache.state, ctx.cu_seqlens, ctx.slots, s.num_heads, s.key_dim, s.value_dim,
                         s.key_dim ** -0.5, write=write)
        y = ops.gated_rmsnorm(o, self.norm, s.norm_eps, gate, s.num_heads, s.value_dim, self.rt.dtype)
        return project(self.rt, y, self.w_out, residual=residual)


class DecayedLinearAttention(Mixer):
    takes_normed = True
    chain_safe = True
    takes_out_dtype = True

    @classmethod
    def kernels(cls, spec):
        return ("recurrent",)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if len(s.decay) != s.num_heads:
            raise ValueError(f"{len(s.decay)} decays for {s.num_heads} heads")
        if s.activation not in (None, "silu") or s.gate_activation not in ("sigmoid", "silu"):
            raise ValueError(f"unknown activation {s.activation!r} or gate activation {s.gate_activation!r}")
        self.w_in = self.w_out = self.norm = self.decay = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        c, hd, hv = s.hidden_size, s.num_heads * s.key_dim, s.num_heads * s.value_dim
        p = {
            self._n("q"): Param((hd, c)),
            self._n("k"): Param((hd, c)),
            self._n("v"): Param((hv, c)),
            self._n("g"): Param((hv, c)),
            self._n("o"): Param((c, hv)),
        }
        if getattr(s, "norm_weight", True):
            p[self._n("norm")] = Param((hv if s.whole_norm else s.value_dim,), role="vector", mean=1.0)
        return p

    def load(self, get):
        self.w_in = stack_rows([get(self._n(n)) for n in ("q", "k", "v", "g")])
        self.norm = get(self._n("norm")) if getattr(self.spec, "norm_weight", True) else None
        self.w_out = get(self._n("o"))
        # the decays are constants of the configuration, kept as float32 (the recurrence's own precision)
        self.decay = torch.tensor([float(d) for d in self.spec.decay], dtype=torch.float64).to(
            device=self.w_out.device, dtype=torch.float32)

    def cache(self):
        s = self.spec
        return StateSpec((s.num_heads, s.value_dim, s.key_dim), torch.float32)  # S transposed, as the scan kernels keep it

    def core(self, proj, ctx, cache, write=True, out=None, out_scale=1.0):
        """From the input product ``proj`` [N, rows of w_in] to what the output product reads, times ``out_scale``."""
        s, ops = self.spec, self.rt.ops
        hd, hv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        q, k, v = proj[:, :hd], proj[:, hd : 2 * hd], proj[:, 2 * hd : 2 * hd + hv]
        gate = proj[:, 2 * hd + hv : 2 * hd + 2 * hv]
        o = ops.decay_scan(q, k, v, self.decay, cache.state, ctx.cu_seqlens, ctx.slots, s.num_heads, s.key_dim, s.value_dim,
                           s.q_scale, activation=s.activation, write=write, longest=getattr(ctx, "max_query_len", None))
        heads, width = (1, hv) if s.whole_norm else (s.num_heads, s.value_dim)
        return ops.gated_rmsnorm(o, self.norm, s.norm_eps, gate, heads, width, self.rt.dtype,
                                 gate_activation=s.gate_activation, out=out, out_scale=out_scale)

    def forward(self, x, ctx, cache=None, residual=None, write=True, out_dtype=None):
        y = self.core(project(self.rt, x, self.w_in), ctx, cache, write)
        return project(self.rt, y, self.w_out, out_dtype=out_dtype, residual=residual)


class GatedDelta(Mixer):
    takes_normed = True
    chain_safe = True

    @classmethod
    def kernels(cls, spec):
        return ("recurrent",)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} heads are not a multiple of {s.num_kv_heads} query/key heads")
        if not 1 <= s.conv_kernel <= 64:
            raise ValueError(f"conv_kernel {s.conv_kernel} must be from 1 to 64")
        self.channels = 2 * s.num_kv_heads * s.key_dim + s.num_heads * s.value_dim  # what the convolution runs over
        self.w_in = self.w_out = self.taps = self.a_log = self.dt_bias = self.norm = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        c, gd, hv, l = s.hidden_size, s.num_kv_heads * s.key_dim, s.num_heads * s.value_dim, s.conv_kernel
        return {
            self._n("q"): Param((gd, c)),
            self._n("q.conv"): Param((gd, l), role="vector", mean=1.0 / l),
            self._n("k"): Param((gd, c)),
            self._n("k.conv"): Param((gd, l), role="vector", mean=1.0 / l),
            self._n("v"): Param((hv, c)),
            self._n("v.conv"): Param((hv, l), role="vector", mean=1.0 / l),
            self._n("b"): Param((s.num_heads, c)),
            self._n("a"): Param((s.num_heads, c)),
            self._n("A_log"): Param((s.num_heads,), role="vector"),
            self._n("dt_bias"): Param((s.num_heads,), role="vector"),
            self._n("g"): Param((hv, c)),
            self._n("norm"): Param((s.value_dim,), role="vector", mean=1.0),
            self._n("o"): Param((c, hv)),
        }

    def load(self, get):
        self.w_in = stack_rows([get(self._n(n)) for n in ("q", "k", "v", "b", "a", "g")])
        self.taps = torch.cat([get(self._n(n)) for n in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = get(self._n("A_log")), get(self._n("dt_bias"))
        self.norm = get(self._n("norm"))
        self.w_out = get(self._n("o"))

    def cache(self):
        """One float32 row per slot: S transposed [heads, value_dim, key_dim], then the convolution's last inputs
        [taps - 1, channels]; the row's length is rounded up to 4 floats so that every slot's S starts on 16 bytes."""
        s = self.spec
        words = s.num_heads * s.key_dim * s.value_dim + (s.conv_kernel - 1) * self.channels
        return StateSpec((-(-words // 4) * 4,), torch.float32)

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        s, ops = self.spec, self.rt.ops
        gd, hv, h, ch = s.num_kv_heads * s.key_dim, s.num_heads * s.value_dim, s.num_heads, self.channels
        slots = cache.state.shape[0]
        matrix_words = h * s.value_dim * s.key_dim
        matrix_state = cache.state[:, :matrix_words].view(slots, h, s.value_dim, s.key_dim)
        conv_state = cache.state[:, matrix_words : matrix_words + (s.conv_kernel - 1) * ch].view(slots, s.conv_kernel - 1, ch)
        proj = project(self.rt, x, self.w_in)
        y = ops.causal_conv_silu(proj[:, :ch], self.taps, conv_state, ctx.cu_seqlens, ctx.seq_of_token, ctx.slots, write=write)
        beta, g = ops.delta_prep(y, s.num_kv_heads, s.key_dim, s.key_dim ** -0.5, s.unit_eps, proj[:, ch : ch + h],
                                 proj[:, ch + h : ch + 2 * h], self.a_log, self.dt_bias)
        o = ops.delta_scan(y[:, :gd], y[:, gd : 2 * gd], y[:, 2 * gd :], beta, g, matrix_state, ctx.cu_seqlens, ctx.slots,
                           h, s.num_kv_heads, s.key_dim, s.value_dim, write=write)
        out = ops.gated_rmsnorm(o, self.norm, s.norm_eps, proj[:, ch + 2 * h : ch + 2 * h + hv], h, s.value_dim, self.rt.dtype)
        return project(self.rt, out, self.w_out, residual=residual)


register_mixer("gated_linear_attention", GatedLinearAttention)
register_mixer("gated_delta", GatedDelta)
register_mixer("decayed_linear_attention", DecayedLinearAttention)
