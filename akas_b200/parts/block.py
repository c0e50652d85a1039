"""A block: a mixer and (unless the layer has none) a feed-forward, each behind its norm, around a float32 residual stream.

``pre_norm`` (the only arrangement LFM2 uses, src/akas/models/lfm2/_composition.py:189,308-309,356
in kreasof-ai/akas): h += mixer(norm(h)); h += ffn(norm(h)). ``parallel``: one norm n = norm(h) that the mixer and
the feed-forward both read, h += m * (s1 * mixer(n) + s2 * ffn(n)) with a constant m and a learned scale per channel
for each sublayer (the two results are float32 and meet the residual stream in one kernel). ``sandwich``: a norm in
front of and a norm behind each sublayer, h += post(mixer(norm(h))); h += post(ffn(norm(h))), the sublayers' results
float32, the second norm and the sum one kernel where the norm offers that (``add_to``). Other arrangements are
added to ``ARRANGEMENTS`` as functions of (block, h, ctx, cache, write).
"""

from __future__ import annotations

import torch

from .base import Param, Runtime, build_part, load_norm, norm_params


def _normed(norm, part, h):
    """The norm's output for ``part``: left to the part's first product when both sides can do that."""
    if getattr(part, "takes_normed", False) and hasattr(norm, "lazy"):
        return norm.lazy(h)
    return norm.forward(h)


def _pre_norm(block, h, ctx, cache, write):
    h = block.mixer.forward(_normed(block.mixer_norm, block.mixer, h), ctx, cache, residual=h, write=write)
    if block.ffn is None:
        return h
    return block.ffn.forward(_normed(block.ffn_norm, block.ffn, h), ctx, residual=h)


def _float32_result(part, *args, **kwargs):
    """A sublayer's result without a residual, in float32: asked of the part where it can say so, else widened."""
    if getattr(part, "takes_out_dtype", False):
        return part.forward(*args, out_dtype=torch.float32, **kwargs)
    return part.forward(*args, **kwargs).to(torch.float32)


def _parallel(block, h, ctx, cache, write):
    n = block.mixer_norm.forward(h)
    a = _float32_result(block.mixer, n, ctx, cache, residual=None, write=write)
    if hasattr(block.ffn, "forward_update"):  # the feed-forward's last kernel does the block's update itself
        return block.ffn.forward_update(n, ctx, h, a, block.mixer_scale, block.ffn_scale, block.spec.residual_multiplier)
    b = None if block.ffn is None else _float32_result(block.ffn, n, ctx, residual=None)
    return block.mixer.rt.ops.scaled_add(h, a, block.mixer_scale, b, block.ffn_scale, block.spec.residual_multiplier)


def _add_normed(norm, y, h, ops):
    """h += norm(y) on the float32 stream, by the norm's own kernel where it has one that adds."""
    if hasattr(norm, "add_to"):
        return norm.add_to(y, h)
    return ops.scaled_add(h, norm.forward(y, out_dtype=torch.float32), None, None, None, 1.0)


def _sandwich(block, h, ctx, cache, write):
    ops = block.mixer.rt.ops
    y = _float32_result(block.mixer, _normed(block.mixer_norm, block.mixer, h), ctx, cache, residual=None, write=write)
    h = _add_normed(block.mixer_post_norm, y, h, ops)
    if block.ffn is None:
        return h
    y = _float32_result(block.ffn, _normed(block.ffn_norm, block.ffn, h), ctx, residual=None)
    return _add_normed(block.ffn_post_norm, y, h, ops)


ARRANGEMENTS = {"pre_norm": _pre_norm, "parallel": _parallel, "sandwich": _sandwich}


class Block:
    def __init__(self, spec, runtime: Runtime):
        if spec.arrangement not in ARRANGEMENTS:
            raise KeyError(f"unknown block arrangement {spec.arrangement!r}; known: {sorted(ARRANGEMENTS)}")
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime)
        self.mixer_post_norm = build_part("norm", getattr(spec, "mixer_post_norm", None), runtime)
        self.ffn_post_norm = build_part("norm", getattr(spec, "ffn_post_norm", None) if self.ffn is not None else None, runtime)
        if spec.arrangement == "sandwich" and (self.mixer_post_norm is None or (self.ffn is not None and self.ffn_post_norm is None)):
            raise ValueError("the sandwich arrangement needs a norm behind each sublayer")
        self._run = ARRANGEMENTS[spec.arrangement]
        self.mixer_scale = self.ffn_scale = None  # the parallel arrangement's scales per channel, where the layer names them
        # Whether every part of the block reaches its tensors through the runtime's operations only (see Part.chain_safe)
        self.chain_safe = all(getattr(part, "chain_safe", False)
                              for part in (self.mixer, self.ffn, self.mixer_norm, self.ffn_norm, self.mixer_post_norm,
                                           self.ffn_post_norm) if part is not None)

    def params(self):
        """Checkpoint name -> Param for everything this block holds."""
        s = self.spec
        out = {s.mixer_prefix + k: v for k, v in self.mixer.params().items()}
        if self.ffn is not None:
            out.update({s.ffn_prefix + k: v for k, v in self.ffn.params().items()})
        norm = norm_params(self.mixer_norm, s.mixer_norm_name)
        out.update(norm)
        norm_param = norm[s.mixer_norm_name]
        width = norm_param.shape
        if s.mixer_scale_name is not None:
            out[s.mixer_scale_name] = Param(width, role="vector", mean=1.0)
        if s.ffn_scale_name is not None:
            # (a layer without a feed-forward: a checkpoint may still carry the scale that would follow one)
            out[s.ffn_scale_name] = Param(width, role="vector", mean=1.0, optional=self.ffn is None)
        if self.ffn is not None and self.ffn_norm is not None:
            out.update(norm_params(self.ffn_norm, s.ffn_norm_name))
        elif self.ffn is not None:
            pass  # an arrangement in which the feed-forward reads the mixer's norm
        elif s.ffn_norm_name is not None:
            # a layer without a feed-forward: a checkpoint may still carry the norm that would precede one
            for name, param in norm_params(self.mixer_norm, s.ffn_norm_name).items():
                out[name] = Param(param.shape, role=param.role, optional=True, mean=param.mean)
        if self.mixer_post_norm is not None:
            out.update(norm_params(self.mixer_post_norm, s.mixer_post_norm_name))
        if self.ffn_post_norm is not None:
            out.update(norm_params(self.ffn_post_norm, s.ffn_post_norm_name))
        elif self.ffn is None and self.mixer_post_norm is not None and getattr(s, "ffn_post_norm_name", None) is not None:
            # a layer without a feed-forward: a checkpoint may still carry the norm that would follow one
            for name, param in norm_params(self.mixer_post_norm, s.ffn_post_norm_name).items():
                out[name] = Param(param.shape, role=param.role, optional=True, mean=param.mean)
        return out

    def load(self, get):
        s = self.spec
        self.mixer.load(lambda name: get(s.mixer_prefix + name))
        load_norm(self.mixer_norm, s.mixer_norm_name, get)
        if self.ffn is not None:
            self.ffn.load(lambda name: get(s.ffn_prefix + name))
            if self.ffn_norm is not None:
                load_norm(self.ffn_norm, s.ffn_norm_name, get)
        if self.mixer_post_norm is not None:
            load_norm(self.mixer_post_norm, s.mixer_post_norm_name, get)
        if self.ffn_post_norm is not None:
            load_norm(self.ffn_post_norm, s.ffn_post_norm_name, get)
        if s.mixer_scale_name is not None:
            self.mixer_scale = get(s.mixer_scale_name)
        if s.ffn_scale_name is not None and self.ffn is not None:
            self.ffn_scale = get(s.ffn_scale_name)

    def forward(self, h, ctx, cache=None, write=True):
        return self._run(self, h, ctx, cache, write)
