"""Grouped-query attention over the paged cache.

In order (src/akas/models/lfm2/_composition.py:234-307 in kreasof-ai/akas): one
product for q, k and v (their three matrices are stacked at load); RMSNorm of each
head of q and k over head_dim, then the position encoding of q and k, and the
write of k and v into the pages at each token's absolute position (one kernel);
attention of every query over the keys of its own request up to its own position,
read from the pages, so a portion of a prompt attends to what earlier steps left
and to itself; the output product, added to the residual.

A layer whose spec asks for more than that (value heads of another size than the keys', a capped score, a
logarithmic distance penalty, first tokens kept behind the window, a sink in the softmax's denominator (exp(0) or a
learned logit per head), a gate per head on the output, values that are the keys as projected, rotary pairs of
neighbouring channels, biases on q, k and v, no keys and values of its own but another layer's cache) runs the same
steps on the general kernels: one product for q, k, v and the gate's
logits, QK-norm, rotation and page write (``ops.qk_norm_store``), attention with the options as arguments
(``ops.attention_general``), the output product. ``core`` is that sequence without the two products, for a mixer
that stacks this one's matrices with its neighbours' (``parts/parallel.py``).
"""

from __future__ import annotations

import torch

from .base import Mixer, PagedKVSpec, Param, build_part, project, register_mixer, renamed, stack_rows


class Attention(Mixer):
    takes_normed = True
    chain_safe = True
    shares_cache = True
    takes_out_dtype = True

    @classmethod
    def kernels(cls, spec):
        if not getattr(spec, "general", False):
            return ("attention",)
        return ("attention_general", "rope") if spec.position is not None else ("attention_general",)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} heads are not a multiple of {s.num_kv_heads} key/value heads")
        self.general = bool(getattr(s, "general", False))
        if not self.general and (s.head_dim % 16 or s.head_dim > 256):
            raise ValueError(f"head_dim {s.head_dim} must be a multiple of 16, at most 256")
        if s.sink not in (False, True, "learned"):
            raise ValueError(f"unknown sink {s.sink!r}; known: False, True, 'learned'")
        if getattr(s, "values_are_keys", False) and s.value_dim != s.head_dim:
            raise ValueError(f"values that are the keys have the keys' size: {s.value_dim} is not {s.head_dim}")
        if self.general and getattr(s, "gate", None) not in (None, "head", "channel"):
            raise ValueError(f"unknown output gate {s.gate!r}; known: 'head', 'channel'")
        if self.general and s.keep_first and not s.window:
            raise ValueError("keep_first needs a window")
        self.own_kv = bool(getattr(s, "own_kv", True))
        self.biased = bool(getattr(s, "bias", False))
        if not self.own_kv and getattr(s, "values_are_keys", False):
            raise ValueError("a layer without keys of its own has no values that are its keys")
        self.q_norm = build_part("norm", s.qk_norm, runtime)
        self.k_norm = build_part("norm", s.qk_norm, runtime)
        self.position = build_part("position", s.position, runtime)
        self.scale = s.scale if s.scale is not None else s.head_dim ** -0.5
        if self.general and self.position is not None and not hasattr(self.position, "tables"):
            raise ValueError("the general attention kernels take a position encoding by rotary tables only")
        self.w_qkv = None
        self.w_out = None
        self.r1 = self.r2 = self.sinks = self.bias = None

    def _n(self, local):
        return renamed(self.spec, local)

    def _gate_rows(self) -> int:
        """How many logits the output gate has per token: one per head, or one per channel of the concatenated heads."""
        s = self.spec
        return {None: 0, "head": s.num_heads, "channel": s.num_heads * s.value_dim}[s.gate]

    def params(self):
        s = self.spec
        vd = s.value_dim if self.general else s.head_dim
        p = {
            self._n("q_proj.weight"): Param((s.num_heads * s.head_dim, s.hidden_size)),
            self._n("k_proj.weight"): Param((s.num_kv_heads * s.head_dim, s.hidden_size)),
            self._n("v_proj.weight"): Param((s.num_kv_heads * vd, s.hidden_size)),
            self._n("out_proj.weight"): Param((s.hidden_size, s.num_heads * vd)),
        }
        if self.general and s.values_are_keys:
            del p[self._n("v_proj.weight")]
        if not self.own_kv:
            p.pop(self._n("k_proj.weight"))
            p.pop(self._n("v_proj.weight"), None)
        if self.biased:
            for local in ("q_proj.weight", "k_proj.weight", "v_proj.weight"):
                if self._n(local) in p:
                    p[self._n(local) + ".b"] = Param((p[self._n(local)].shape[0],), role="vector")
        if self.general and s.sink == "learned":
            p[self._n("sink")] = Param((s.num_heads,), role="vector")
        if self.general and s.gate is not None:
            p[self._n("gate.weight")] = Param((self._gate_rows(), s.hidden_size))
        if self.general and s.distance_bias:
            p[self._n("r1")] = Param((s.num_heads,), role="vector")
            p[self._n("r2")] = Param((s.num_heads,), role="vector", mean=0.5)
        if self.q_norm is not None:
            (norm_param,) = self.q_norm.params().values()
            p[self._n("q_norm.weight")] = norm_param
            p[self._n("k_norm.weight")] = norm_param
        return p

    def load(self, get):
        if self.general:
            names = [self._n("q_proj.weight")]
            if self.own_kv:
                names.append(self._n("k_proj.weight"))
                if not self.spec.values_are_keys:
                    names.append(self._n("v_proj.weight"))
            parts = [get(name) for name in names]
            if self.spec.gate is not None:
                parts.append(get(self._n("gate.weight")))
            self.w_qkv = stack_rows(parts)
            if self.biased:
                self.bias = torch.cat([get(name + ".b") for name in names]).contiguous()
            if self.spec.sink == "learned":
                self.sinks = get(self._n("sink"))
            if self.spec.distance_bias:
                self.r1, self.r2 = get(self._n("r1")), get(self._n("r2"))
        else:
            self.w_qkv = torch.cat(
                [get(self._n("q_proj.weight")), get(self._n("k_proj.weight")), get(self._n("v_proj.weight"))], dim=0
            ).contiguous()
        self.w_out = get(self._n("out_proj.weight"))
        if self.q_norm is not None:
            self.q_norm.weight = get(self._n("q_norm.weight"))
            self.k_norm.weight = get(self._n("k_norm.weight"))

    def cache(self):
        s = self.spec
        if not self.own_kv:
            raise ValueError("this attention layer keeps no keys and values: the run order must give it another layer's cache")
        if self.general:
            return PagedKVSpec(s.num_kv_heads, s.head_dim, s.window, keep_first=s.keep_first if s.window else 0,
                               v_head_dim=s.value_dim)
        return PagedKVSpec(s.num_kv_heads, s.head_dim, s.window)

    @property
    def w_in(self):
        """The stacked input matrices (general layers): what ``core`` wants the product of."""
        return self.w_qkv

    def core(self, proj, ctx, cache, write=True, out=None, out_scale=1.0):
        """Everything between the input product ``proj`` [N, rows of w_in] and the output product: the heads'
        outputs [N, heads * value_dim] times ``out_scale``, written to ``out`` where that is given (a view whose rows
        may be part of wider rows)."""
        if not self.general:
            raise ValueError("core() is the general layers' sequence")
        s, ops = self.spec, self.rt.ops
        if not self.own_kv and write:
            raise ValueError("a layer without keys and values of its own writes no cache")
        nq = s.num_heads * s.head_dim
        nk = s.num_kv_heads * s.head_dim if self.own_kv else 0
        nv = 0 if s.values_are_keys or not self.own_kv else s.num_kv_heads * s.value_dim
        q = proj[:, :nq]
        k = proj[:, nq : nq + nk] if self.own_kv else q  # (with nothing to write, k and v are not read)
        v = k if s.values_are_keys or not self.own_kv else proj[:, nq + nk : nq + nk + nv]
        gate = proj[:, nq + nk + nv : nq + nk + nv + self._gate_rows()] if s.gate is not None else None
        norm = self.q_norm.spec if self.q_norm is not None else None
        if norm is not None and norm.zero_centered:
            raise ValueError("the general attention kernels take a plain QK-norm weight")
        table = ctx.block_table(cache.group)
        rotary = {}
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary = dict(cos=cos, sin=sin, interleaved=self.position.interleaved)
        if self.bias is not None:
            rotary.update(q_bias=self.bias[:nq], k_bias=self.bias[nq : nq + nk] if nk else None,
                          v_bias=self.bias[nq + nk : nq + nk + nv] if nv else None)
        qn = ops.qk_norm_store(
            q, k, v, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim,
            self.q_norm.weight if norm else None, self.k_norm.weight if norm else None, norm.eps if norm else 0.0,
            cache.k, cache.v, table, ctx.seq_of_token, ctx.positions, cache.page_size, write=write, **rotary,
        )
        more = {}
        if self.sinks is not None:
            more["sinks"] = self.sinks
        if out is not None:
            more["out"] = out
        if out_scale != 1.0:
            more["out_scale"] = out_scale
        if s.gate == "channel":
            more["gate_channels"] = True
        return ops.attention_general(
            qn, cache.k, cache.v, table, ctx.seq_of_token, ctx.positions, self.scale, s.window, s.keep_first,
            s.softcap, self.r1, self.r2, s.sink is True, gate, cache.page_size, ctx, **more,
        )

    def _forward_general(self, x, ctx, cache, residual, write, out_dtype=None):
        # with biases the product leaves float32, so that product plus bias is rounded once (by the kernel that adds it)
        proj = project(self.rt, x, self.w_qkv, out_dtype=torch.float32 if self.bias is not None else None)
        out = self.core(proj, ctx, cache, write)
        return project(self.rt, out, self.w_out, out_dtype=out_dtype, residual=residual)

    def forward(self, x, ctx, cache=None, residual=None, write=True, out_dtype=None):
        s, ops = self.spec, self.rt.ops
        if self.general:
            return self._forward_general(x, ctx, cache, residual, write, out_dtype)
        if out_dtype is not None and residual is None:
            return self.forward(x, ctx, cache, None, write).to(out_dtype)
        qkv = project(self.rt, x, self.w_qkv)
        fused = self.position is None or hasattr(self.position, "tables")
        cos = sin = None
        if self.position is not None and fused:
            cos, sin = self.position.tables(ctx)
        norm = self.q_norm.spec if self.q_norm is not None else None
        if fused and ctx.decode_only and hasattr(ops, "qkv_decode_attention"):
            # a decode step: everything between the qkv product and the output product as one kernel, where there is one
            out = ops.qkv_decode_attention(
                qkv, s.num_heads, s.num_kv_heads, s.head_dim,
                self.q_norm.weight if norm else None, self.k_norm.weight if norm else None,
                norm.eps if norm else 0.0, bool(norm and norm.zero_centered), cos, sin, cache.k, cache.v,
                ctx.block_table(cache.group), ctx.seq_of_token, ctx.positions, self.scale, s.window, cache.page_size,
                ctx, write=write,
            )
            if out is not None:
                return project(self.rt, out, self.w_out, residual=residual)
        store = write and fused
        q = ops.qk_norm_rope_store(
            qkv, s.num_heads, s.num_kv_heads, s.head_dim,
            self.q_norm.weight if norm else None, self.k_norm.weight if norm else None,
            norm.eps if norm else 0.0, bool(norm and norm.zero_centered), cos, sin,
            cache.k if store else None, cache.v if store else None,
            ctx.block_table(cache.group), ctx.seq_of_token, ctx.positions, cache.page_size,
        )
        if not fused:
            # A position encoding without rotary tables rewrites q and k itself; k and v go to the pages after it.
            k = qkv[:, s.num_heads * s.head_dim : (s.num_heads + s.num_kv_heads) * s.head_dim]
            q, k = self.position.apply(q, k, ctx)
            if write:
                v = qkv[:, (s.num_heads + s.num_kv_heads) * s.head_dim :]
                ops.kv_store(k, v, cache.k, cache.v, ctx.block_table(cache.group), ctx.seq_of_token,
                             ctx.positions, cache.page_size)
        out = ops.paged_attention(
            q, cache.k, cache.v, ctx.block_table(cache.group), ctx.seq_of_token, ctx.positions,
            self.scale, s.window, cache.page_size, ctx,
        )
        return project(self.rt, out, self.w_out, residual=residual)


register_mixer("attention", Attention)
