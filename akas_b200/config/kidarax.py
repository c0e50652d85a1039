"""Typed configuration of the Kidarax decoder, read from its own config.json keys.

A Kidarax model is a list of layers around a float32 residual stream. Every norm is a Dynamic Tanh
(tanh(alpha x) * w + b, no statistics), and every sublayer stands between two of them:
x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))). A layer's mixer is one of three. ``retention``: linear
attention with one constant decay per head, no softmax and no denominator, keys times dim^(-1/2), every head's
read-out divided by its root mean square, the heads times silu(W_g h). ``attention``: causal grouped-query softmax
attention with biased projections, rotate-half rotary positions on the first ``rot.dims`` channels of a head with
every rate divided by ``rot.scaling.factor``, the score scale of the configuration, and the concatenated heads times
sigmoid(W_g h). ``latent_attention``: keys and values through one normed low-rank latent plus a rotated key part that
all heads share, queries a plain projection, rates blended by the pair's index (``rot.scaling`` with ``original``,
``fast``, ``slow``) and tables scaled by 0.1 ln(factor) + 1, a learned sink per head in the softmax's denominator,
head h's output times sigmoid(W_g h)_h. The feed-forward is ``dense`` (W_down relu(W_up h)^2), ``moe`` (a sigmoid
router in float32, the ``top`` largest scores, each expert run on its weight times the token's row, and one expert
that every token passes, times sigmoid(W_sg h)), or none. ``loop`` runs the layers ``start .. stop - 1`` ``times``
times in a row with the same weights, every pass with a cache of its own, and before every pass but the first the
embedding's output is added to the stream. The head is the embedding; the logits are multiplied by ``logit_scale``.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b`` (each with ``.alpha``,
``.b``), ``l<i>.mix.{q,k,v,g,o}`` (attention: ``q.b``, ``k.b``, ``v.b``), ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,g,o}``,
``l<i>.mlp.{up,down}``, ``l<i>.mlp.{router,e<j>.{gate,up,down},shared.{gate,up,down,sg}}``, ``final.norm``.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple

from .girelix import _freeze, _int, _number, _thaw
from .lfm2 import ConfigError
from .specs import (
    AttentionSpec,
    DecayedLinearAttentionSpec,
    DynamicTanhSpec,
    LatentAttentionSpec,
    LayerSpec,
    MLPSpec,
    ModelSpec,
    RopeSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
)

ARCHITECTURE = "Kidarax"
MIXER_TYPES = ("retention", "attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _rot(where: str, m: Mapping[str, Any], most: int, blended: bool) -> None:
    rot = m.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"{where}.rot must be an object")
    dims = _int(where + ".rot", rot, "dims", least=0)
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot.dims {dims} must be even and at most {most}")
    base = _number(where + ".rot", rot, "base")
    scaling = rot.get("scaling")
    if scaling is not None:
        w = where + ".rot.scaling"
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"{w} must be an object")
        _number(w, scaling, "factor")
        if blended and any(key in scaling for key in ("original", "fast", "slow")):
            for key in ("original", "fast", "slow"):
                _number(w, scaling, key)
            if base == 1.0:
                raise ConfigError(f"{where}.rot.base 1 leaves the blend of the rates undefined")


def _rope(head: int, rot: Mapping[str, Any], dims: int, blended: bool) -> Optional[RopeSpec]:
    """The rotation of the first ``dims`` channels of a head of ``head`` channels; the rates are divided by the
    scaling's factor, or (``blended``) blended by the pair's index with both tables scaled."""
    if not dims:
        return None
    s = rot.get("scaling")
    if s is None:
        return RopeSpec(head, float(rot["base"]), dims)
    factor = float(s["factor"])
    if not blended or "original" not in s:  # (a scaling that names a factor only stretches evenly, whatever the mixer)
        return RopeSpec(head, float(rot["base"]), dims, linear_factor=factor)
    return RopeSpec(head, float(rot["base"]), dims, blend=(factor, float(s["original"]), float(s["fast"]), float(s["slow"])),
                    amplitude=0.1 * math.log(factor) + 1.0)


@dataclass(frozen=True)
class KidaraxLayer:
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
class KidaraxConfig:
    width: int
    vocab: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[KidaraxLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "KidaraxConfig":
        if data.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {ARCHITECTURE!r}")
        width = _int("config", data, "width")
        vocab = _int("config", data, "vocab")
        eps = _number("norm", data.get("norm") or {}, "eps")
        scale = 1.0 if data.get("logit_scale") is None else _number("config", data, "logit_scale", positive=False)
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
            getattr(cls, "_check_" + kind)(where + ".mixer", m)
            mlp = entry.get("mlp")
            if mlp is not None:
                cls._check_mlp(where + ".mlp", mlp)
            layers.append(KidaraxLayer(kind, _freeze(m), None if mlp is None else _freeze(mlp)))
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("loop must be an object")
            start, stop = _int("loop", loop, "start", least=0), _int("loop", loop, "stop", least=0)
            times = _int("loop", loop, "times", least=1)
            if not start <= stop <= len(layers):
                raise ConfigError(f"loop: start {start} .. stop {stop} is no stretch of {len(layers)} layers")
            loop = (start, stop, times)
        eos = data.get("eos_token_id")
        return cls(width=width, vocab=vocab, norm_eps=eps, logit_scale=scale, layers=tuple(layers), loop=loop,
                   eos_token_id=eos if type(eos) is int else None)

    @staticmethod
    def _check_retention(where: str, m: Mapping[str, Any]) -> None:
        heads = _int(where, m, "heads")
        _int(where, m, "dim"), _int(where, m, "vdim")
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads:
            raise ConfigError(f"{where}.decay must list one number for each of the {heads} heads")
        for a in decay:
            if isinstance(a, bool) or not isinstance(a, (int, float)) or not math.isfinite(a) or not 0.0 <= a <= 1.0:
                raise ConfigError(f"{where}.decay: {a!r} is no number from 0 to 1")

    @staticmethod
    def _check_attention(where: str, m: Mapping[str, Any]) -> None:
        heads, dim = _int(where, m, "heads"), _int(where, m, "dim")
        if heads % _int(where, m, "kv_heads"):
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {m['kv_heads']} kv_heads")
        _int(where, m, "vdim")
        _number(where, m, "scale")
        _rot(where, m, dim, blended=False)

    @staticmethod
    def _check_latent_attention(where: str, m: Mapping[str, Any]) -> None:
        for key in ("heads", "dim", "vdim", "kv_rank"):
            _int(where, m, key)
        rot_dim = _int(where, m, "rot_dim", least=0)
        _number(where, m, "scale")
        _rot(where, m, rot_dim, blended=True)
        if m["rot"]["dims"] != rot_dim:
            raise ConfigError(f"{where}: rot.dims {m['rot']['dims']} must equal rot_dim {rot_dim}, the part that turns")

    @staticmethod
    def _check_mlp(where: str, mlp: Any) -> None:
        kind = mlp.get("kind") if isinstance(mlp, Mapping) else None
        if kind not in MLP_KINDS:
            raise ConfigError(f"{where}.kind {kind!r} is none of {list(MLP_KINDS)}")
        if kind == "dense":
            _int(where, mlp, "ff")
            return
        _int(where + ".expert", mlp.get("expert"), "ff")
        experts = _int(where + ".router", mlp.get("router"), "experts")
        top = _int(where + ".router", mlp.get("router"), "top")
        if top > experts:
            raise ConfigError(f"{where}.router: top {top} exceeds the {experts} experts")
        if mlp.get("shared") is not None:
            _int(where + ".shared", mlp.get("shared"), "ff")

    @classmethod
    def from_json(cls, path) -> "KidaraxConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        """A config.json that reads back as this configuration."""
        data = dict(
            architecture=ARCHITECTURE,
            layers=[dict(type=l.type, mixer=l.mixer_options, mlp=l.mlp_options) for l in self.layers],
            logit_scale=self.logit_scale,
            norm=dict(eps=self.norm_eps),
            vocab=self.vocab,
            width=self.width,
        )
        if self.loop is not None:
            data["loop"] = dict(start=self.loop[0], stop=self.loop[1], times=self.loop[2])
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # ------------------------------------------------------------------ the model it describes

    def mixer_spec(self, layer: KidaraxLayer):
        m, c = layer.mixer_options, self.width
        if layer.type == "retention":
            # S <- a S + (k / sqrt(dim)) v^T, o = S^T q: the constant rides on q, which is the same sum
            return DecayedLinearAttentionSpec(
                c, m["heads"], m["dim"], m["vdim"], tuple(float(a) for a in m["decay"]), self.norm_eps, activation=None,
                whole_norm=False, gate_activation="silu", q_scale=m["dim"] ** -0.5, norm_weight=False,
            )
        rot = m["rot"]
        if layer.type == "attention":
            names = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "out_proj.weight": "o", "gate.weight": "g"}
            return AttentionSpec(
                c, m["heads"], m["kv_heads"], m["dim"], position=_rope(m["dim"], rot, rot["dims"], blended=False),
                scale=float(m["scale"]), v_head_dim=m["vdim"], bias=True, gate="channel", names=names,
            )
        return LatentAttentionSpec(
            c, m["heads"], m["dim"], m["rot_dim"], m["vdim"], None, m["kv_rank"], self.norm_eps, float(m["scale"]),
            position=_rope(m["rot_dim"], rot, m["rot_dim"], blended=True), sink="learned", gate="head",
        )

    def ffn_spec(self, layer: KidaraxLayer):
        mlp = layer.mlp_options
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return MLPSpec(self.width, mlp["ff"], activation="relu2")
        shared = mlp.get("shared")
        return RoutedExpertsSpec(
            self.width, mlp["expert"]["ff"], mlp["router"]["experts"], 0, mlp["router"]["top"], scoring="sigmoid",
            correction=False, renormalize=False, weight_on="input", shared_size=None if shared is None else shared["ff"],
            shared_gate=shared is not None,
        )

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        """One entry per layer run; a layer inside the loop runs ``times`` times, each time with a cache of its own,
        and the first layer of every pass but the first has the embedding's output added in front of it."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(ScheduleEntry(i) for i in range(n))
        start, stop, times = self.loop
        order = [ScheduleEntry(i) for i in range(start)]
        for turn in range(times):
            order += [ScheduleEntry(i, add_embedding=turn > 0 and i == start) for i in range(start, stop)]
        return tuple(order + [ScheduleEntry(i) for i in range(stop, n)])

    def model_spec(self) -> ModelSpec:
        norm = DynamicTanhSpec(self.width)
        layers = []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            ffn = self.ffn_spec(layer)
            layers.append(LayerSpec(
                mixer=self.mixer_spec(layer),
                ffn=ffn,
                mixer_norm=norm,
                ffn_norm=None if ffn is None else norm,
                mixer_prefix=prefix + "mix.",
                ffn_prefix=prefix + "mlp.",
                mixer_norm_name=prefix + "norm1",
                ffn_norm_name=prefix + "norm2",
                arrangement="sandwich",
                mixer_post_norm=norm,
                ffn_post_norm=None if ffn is None else norm,
                mixer_post_norm_name=prefix + "norm1b",
                ffn_post_norm_name=prefix + "norm2b",
            ))
        return ModelSpec(
            architecture=ARCHITECTURE,
            hidden_size=self.width,
            vocab_size=self.vocab,
            layers=tuple(layers),
            final_norm=norm,
            embedding_name="embed",
            final_norm_name="final.norm",
            head_name=None,
            schedule=self.run_order(),
            logit_scale=self.logit_scale,
        )
