"""Typed configuration of the Penopel decoder, read from its own config.json keys.

A Penopel model is a list of pre-norm layers around a float32 residual stream. Every norm is a Dynamic Tanh
(tanh(alpha x) * w + b, no statistics). A layer's mixer is one of two: ``attention``, causal grouped-query attention
with biased projections, rotate-half rotary positions on the first ``rot.dims`` channels of a head (optionally with
long waves slowed, ``rot.scaling``), a softmax with one added to its denominator, and, with ``kv_from: j``, no key and
value projections of its own but layer j's cache; or ``latent_attention``, attention through low-rank latents over a
sliding window with a learned sink per head and a sigmoid gate on the heads' outputs, of which only the latent and a
shared rotated key part are cached. The feed-forward is a gated one with the tanh form of gelu and biases. The
embedding is scaled, and the logits pass a tanh cap. config.json lists the layers one by one
(``layers[i] = {"type", "mixer", "mlp"}``), so every layer may have sizes of its own and a layer may have no
feed-forward.

Checkpoint names: ``embed``, ``l<i>.norm1`` (``.alpha``, ``.b``), ``l<i>.norm2``, ``l<i>.mix.{q,k,v}`` (``.b``),
``l<i>.mix.o``, ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}``, ``l<i>.mlp.{gate,up,down}`` (``.b``),
``final.norm``, ``head``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple

from .girelix import _freeze, _int, _number, _thaw
from .lfm2 import ConfigError
from .specs import (
    AttentionSpec,
    DynamicTanhSpec,
    GatedMLPSpec,
    LatentAttentionSpec,
    LayerSpec,
    ModelSpec,
    RopeSpec,
    ScheduleEntry,
)

ARCHITECTURE = "Penopel"
MIXER_TYPES = ("attention", "latent_attention")


def _rot(where: str, m: Mapping[str, Any], most: int) -> None:
    rot = m.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"{where}.rot must be an object")
    dims = _int(where + ".rot", rot, "dims", least=0)
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot.dims {dims} must be even and at most {most}")
    _number(where + ".rot", rot, "base")
    scaling = rot.get("scaling")
    if scaling is not None:
        w = where + ".rot.scaling"
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"{w} must be an object")
        _number(w, scaling, "factor"), _number(w, scaling, "original")
        low, high = _number(w, scaling, "low"), _number(w, scaling, "high")
        if high <= low:
            raise ConfigError(f"{w}: high {high} must exceed low {low}")


def _rope(head: int, rot: Mapping[str, Any], dims: int, interleaved: bool) -> Optional[RopeSpec]:
    if not dims:
        return None
    s = rot.get("scaling")
    scaling = None if s is None else (float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"]))
    return RopeSpec(head, float(rot["base"]), dims, interleaved=interleaved, scaling=scaling)


@dataclass(frozen=True)
class PenopelLayer:
    """One entry of ``layers``: its type and what config.json gives for its mixer and its feed-forward (None: none),
    kept as nested tuples so that the layer can be hashed."""

    type: str
    mixer: tuple
    mlp: Optional[tuple]

    @property
    def mixer_options(self) -> dict:
        return _thaw(self.mixer)

    @property
    def mlp_options(self) -> Optional[dict]:
        return None if self.mlp is None else _thaw(self.mlp)


@dataclass(frozen=True)
class PenopelConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: Optional[float]
    layers: Tuple[PenopelLayer, ...]
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "PenopelConfig":
        if data.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {ARCHITECTURE!r}")
        width = _int("config", data, "width")
        vocab = _int("config", data, "vocab")
        eps = _number("norm", data.get("norm") or {}, "eps")
        scale = _number("embedding", data.get("embedding") or {}, "scale", positive=False)
        cap = None if data.get("logit_softcap") is None else _number("config", data, "logit_softcap")
        listed = data.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, Mapping) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}.type {kind!r} is none of {list(MIXER_TYPES)}")
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind == "attention":
                cls._check_attention(where + ".mixer", m, i, listed)
            else:
                cls._check_latent(where + ".mixer", m)
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not 'dense'")
                _int(where + ".mlp", mlp, "ff")
            layers.append(PenopelLayer(kind, _freeze(m), None if mlp is None else _freeze(mlp)))
        eos = data.get("eos_token_id")
        return cls(width=width, vocab=vocab, norm_eps=eps, embedding_scale=scale, logit_softcap=cap, layers=tuple(layers),
                   eos_token_id=eos if type(eos) is int else None)

    @staticmethod
    def _check_attention(where: str, m: Mapping[str, Any], index: int, listed) -> None:
        heads, dim = _int(where, m, "heads"), _int(where, m, "dim")
        if heads % _int(where, m, "kv_heads"):
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {m['kv_heads']} kv_heads")
        _int(where, m, "vdim")
        _number(where, m, "scale")
        _rot(where, m, dim)
        if m.get("kv_from") is not None:
            j = m["kv_from"]
            if type(j) is not int or not 0 <= j < index:
                raise ConfigError(f"{where}.kv_from {j!r} must name an earlier layer")
            other = listed[j]
            theirs = other.get("mixer") if isinstance(other, Mapping) else None
            if other.get("type") != "attention" or not isinstance(theirs, Mapping) or theirs.get("kv_from") is not None:
                raise ConfigError(f"{where}.kv_from {j}: that layer is no attention layer with keys and values of its own")
            for key in ("kv_heads", "dim", "vdim", "rot"):
                if theirs.get(key) != m.get(key):
                    raise ConfigError(f"{where}.kv_from {j}: {key} differs ({m.get(key)!r} here, {theirs.get(key)!r} there)")

    @staticmethod
    def _check_latent(where: str, m: Mapping[str, Any]) -> None:
        for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
            _int(where, m, key)
        rot_dim = _int(where, m, "rot_dim", least=0)
        _number(where, m, "scale")
        _rot(where, m, rot_dim)
        if m["rot"]["dims"] != rot_dim:
            raise ConfigError(f"{where}: rot.dims {m['rot']['dims']} must equal rot_dim {rot_dim}, the part that turns")
        mask = m.get("mask")
        if mask is not None:
            if not isinstance(mask, Mapping):
                raise ConfigError(f"{where}.mask must be an object")
            _int(where + ".mask", mask, "size")

    @classmethod
    def from_json(cls, path) -> "PenopelConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        """A config.json that reads back as this configuration."""
        data = dict(
            architecture=ARCHITECTURE,
            embedding=dict(scale=self.embedding_scale),
            layers=[dict(type=l.type, mixer=l.mixer_options, mlp=l.mlp_options) for l in self.layers],
            norm=dict(eps=self.norm_eps),
            vocab=self.vocab,
            width=self.width,
        )
        if self.logit_softcap is not None:
            data["logit_softcap"] = self.logit_softcap
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # ------------------------------------------------------------------ the model it describes

    def mixer_spec(self, layer: PenopelLayer):
        m, c = layer.mixer_options, self.width
        rot = m["rot"]
        if layer.type == "attention":
            names = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "out_proj.weight": "o"}
            return AttentionSpec(
                c, m["heads"], m["kv_heads"], m["dim"], position=_rope(m["dim"], rot, rot["dims"], interleaved=False),
                scale=float(m["scale"]), v_head_dim=m["vdim"], sink=True, bias=True, own_kv=m.get("kv_from") is None, names=names,
            )
        mask = m.get("mask")
        return LatentAttentionSpec(
            c, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], self.norm_eps, float(m["scale"]),
            position=_rope(m["rot_dim"], rot, m["rot_dim"], interleaved=True), window=None if mask is None else mask["size"],
            sink="learned", gate="channel",
        )

    def model_spec(self) -> ModelSpec:
        norm = DynamicTanhSpec(self.width)
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            mlp = layer.mlp_options
            layers.append(LayerSpec(
                mixer=self.mixer_spec(layer),
                ffn=None if mlp is None else GatedMLPSpec(self.width, mlp["ff"], activation="gelu_tanh", bias=True),
                mixer_norm=norm,
                ffn_norm=None if mlp is None else norm,
                mixer_prefix=prefix + "mix.",
                ffn_prefix=prefix + "mlp.",
                mixer_norm_name=prefix + "norm1",
                ffn_norm_name=prefix + "norm2",
            ))
            # the run order is the layers' order (one schedule entry a layer), so a layer's number names its entry
            schedule.append(ScheduleEntry(i, cache=layer.mixer_options.get("kv_from") if layer.type == "attention" else None))
        return ModelSpec(
            architecture=ARCHITECTURE,
            hidden_size=self.width,
            vocab_size=self.vocab,
            layers=tuple(layers),
            final_norm=norm,
            embedding_name="embed",
            final_norm_name="final.norm",
            head_name="head",
            head_optional=False,
            schedule=tuple(schedule),
            embedding_multiplier=self.embedding_scale,
            logit_softcap=self.logit_softcap,
        )
