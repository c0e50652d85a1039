"""Attention through low-rank latents, computed in the latents' own space.

What the design states per head h (plain key W_uk,h c_j, value W_uv,h c_j of the cached latent c_j) is computed
without ever forming those keys and values:

    score_ij = ((W_uk,h^T q_plain_i) . c_j + q_rot_i . k_rot_j) * scale,   out_i = W_uv,h (sum_j p_ij c_j),

so the cache holds one row [c_j (kv_rank), k_rot_j (rope_dim)] per token, that row is the key of every head and its
first kv_rank channels are the value of every head: attention with ONE key/value head whose group is all the query
heads, which the general attention kernels run with the heads of a token packed into one block (a decode step reads
each cached row once for all heads). The two per-head products around it (``ops.head_linear``) carry the query's
rotation and the output gate in their read-outs.

In order: one product for everything that reads the mixer's input (W_dq, W_dkv and the gate's W_g stacked; float32
out); ``ops.latent_norm_store`` (RMS norm of the query latent; RMS norm of c, rotation of the shared key part, the
row's write into the pages); the query's up product; ``ops.head_linear`` (W_uk,h^T q_plain, rotated q_rot carried
over); ``ops.attention_general`` over the latent pages (window, sink, scale); ``ops.head_linear`` (W_uv,h, times
sigmoid of the gate's logits); the output product, added to the residual.
"""

from __future__ import annotations

import torch

from .base import Mixer, PagedLatentSpec, Param, build_part, project, register_mixer, renamed, stack_rows


class LatentAttention(Mixer):
    takes_normed = True
    chain_safe = True
    shares_cache = True
    takes_out_dtype = True

    @classmethod
    def kernels(cls, spec):
        return ("attention_general", "latent", "rope") if spec.position is not None else ("attention_general", "latent")

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.sink not in (False, True, "learned"):
            raise ValueError(f"unknown sink {s.sink!r}; known: False, True, 'learned'")
        if s.gate not in (None, "channel", "head"):
            raise ValueError(f"unknown output gate {s.gate!r}; known: 'channel', 'head'")
        self.q_rank = s.q_rank or 0  # 0: the queries are a projection of the input itself
        self.position = build_part("position", s.position, runtime)
        if self.position is not None and (not hasattr(self.position, "tables") or s.position.rotary != s.rope_dim):
            raise ValueError("the rotated part turns as a whole, by rotary tables")
        if self.position is None and s.rope_dim:
            raise ValueError(f"a rotated part of {s.rope_dim} channels needs a position encoding")
        self.w_in = self.w_uq = self.w_q = self.w_absorb = self.w_uv = self.w_out = None
        self.q_norm = self.kv_norm = self.sinks = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        c, h = s.hidden_size, s.num_heads
        p = {
            self._n("dq"): Param((self.q_rank, c)),
            self._n("dq.norm"): Param((self.q_rank,), role="vector", mean=1.0),
            self._n("uq"): Param((h * (s.head_dim + s.rope_dim), self.q_rank)),
        } if self.q_rank else {self._n("q"): Param((h * (s.head_dim + s.rope_dim), c))}
        p |= {
            self._n("dkv"): Param((s.kv_rank + s.rope_dim, c)),
            self._n("dkv.norm"): Param((s.kv_rank,), role="vector", mean=1.0),
            self._n("uk"): Param((h * s.head_dim, s.kv_rank)),
            self._n("uv"): Param((h * s.v_head_dim, s.kv_rank)),
            self._n("o"): Param((c, h * s.v_head_dim)),
        }
        if s.sink == "learned":
            p[self._n("sink")] = Param((h,), role="vector")
        if s.gate == "channel":
            p[self._n("g")] = Param((h * s.v_head_dim, c))
        if s.gate == "head":
            p[self._n("g")] = Param((h, c))
        return p

    def load(self, get):
        s = self.spec
        parts = [get(self._n("dq"))] if self.q_rank else []
        parts.append(get(self._n("dkv")))
        if s.gate is not None:
            parts.append(get(self._n("g")))
        self.w_in = stack_rows(parts)
        self.kv_norm = get(self._n("dkv.norm"))
        if self.q_rank:
            self.q_norm, self.w_uq = get(self._n("dq.norm")), get(self._n("uq"))
        else:
            self.w_q = get(self._n("q"))
        # per head [out, in]: W_uk,h^T takes a head's plain query channels to the latent's; W_uv,h the latent to the values
        self.w_absorb = get(self._n("uk")).reshape(s.num_heads, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = get(self._n("uv")).reshape(s.num_heads, s.v_head_dim, s.kv_rank).contiguous()
        self.w_out = get(self._n("o"))
        if s.sink == "learned":
            self.sinks = get(self._n("sink"))

    def cache(self):
        s = self.spec
        return PagedLatentSpec(s.kv_rank + s.rope_dim, s.window)

    def forward(self, x, ctx, cache=None, residual=None, write=True, out_dtype=None):
        s, ops = self.spec, self.rt.ops
        # without a query latent the queries are a product of their own, in the compute dtype (the other leaves float32
        # for the latent's norm)
        q = None if self.q_rank else project(self.rt, x, self.w_q)
        proj = project(self.rt, x, self.w_in, out_dtype=torch.float32)
        cos = sin = None
        interleaved = False
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            interleaved = self.position.interleaved
        table = ctx.block_table(cache.group)
        query_latent = ops.latent_norm_store(
            proj, self.q_rank, s.kv_rank, s.rope_dim, self.q_norm, self.kv_norm, s.norm_eps, cos, sin, interleaved, cache.kv,
            table, ctx.seq_of_token, ctx.positions, cache.page_size, write=write,
        )
        if self.q_rank:
            q = ops.linear(query_latent, self.w_uq)
        q = ops.head_linear(q, self.w_absorb, s.num_heads, cos=cos, sin=sin, interleaved=interleaved)
        more = {"sinks": self.sinks} if self.sinks is not None else {}
        first = self.q_rank + s.kv_rank + s.rope_dim  # where the gate's logits start in the product's rows
        head_gate = None
        if s.gate == "head":
            # one number per head commutes with the head's value product: it rides in attention's read-out
            head_gate = proj[:, first : first + s.num_heads]  # (float32, as the product left them)
        latent = ops.attention_general(
            q, cache.kv, cache.kv, table, ctx.seq_of_token, ctx.positions, s.scale, s.window, 0, None, None, None,
            s.sink is True, head_gate, cache.page_size, ctx, values_in_keys=s.kv_rank, **more,
        )
        gate = None
        if s.gate == "channel":
            gate = proj[:, first : first + s.num_heads * s.v_head_dim]
        out = ops.head_linear(latent, self.w_uv, s.num_heads, gate=gate)
        return project(self.rt, out, self.w_out, out_dtype=out_dtype, residual=residual)


register_mixer("latent_attention", LatentAttention)
