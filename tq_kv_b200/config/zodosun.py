"""Typed configuration of the Zodosun decoder and the builder that turns it
into a `ModelSpec` of parts.

A Zodosun config.json names its architecture with the key `architecture`, its
sizes with `vocab` and `width`, the norm's `eps` and `groups` under `norm`, a
`logit_scale`, and lists its layers one by one: every layer gives its `type`
(which mixer it has), the mixer's sizes and constants under `mixer`, and its
feed-forward under `mlp` (null: the layer has only the mixer).  Layers of
different types may follow one another in any order.

Mixers:
  general_delta   heads x dim; a square float32 state per head (parts/delta_rule.py)
  parallel        two mixers side by side on the same input: `left`, an
                  attention with sigmoid weights (parts/sigmoid_attention.py),
                  and `right`, a state with a constant decay per head
                  (parts/decayed_state.py); their normed results are averaged
                  (parts/side_by_side.py)

Two sizes are not in the configuration but in the tensors' shapes: the inner
width of the delta rule's decay projection and the number of rows of the
attention's distance table.  The optional keys `rank` (of a general_delta
mixer) and `bias_rows` (of a left mixer) give them where there are no tensors
to read them from (random weights); a checkpoint's shapes win otherwise.
Positions have no limit by design; `max_positions` (optional, default 32,768)
bounds the cache an engine plans for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Zodosun"
MODEL_TYPE = "zodosun"
DEFAULT_MAX_POSITIONS = 32768
SINUSOID_BASE = 10000.0          # fixed by the design
UNIT_KEY_EPS = 1e-6              # fixed by the design


def _need(d: dict, key: str, typ, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks the key '{key}'")
    v = d[key]
    if typ is float and isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    if typ is int and isinstance(v, int) and not isinstance(v, bool):
        return int(v)
    if typ is str and isinstance(v, str):
        return v
    if typ is dict and isinstance(v, dict):
        return v
    if typ is list and isinstance(v, list):
        return v
    raise ConfigError(f"config.json: {where}: key '{key}' should be {typ.__name__}, found {v!r}")


def _positive(where: str, **values) -> None:
    for name, v in values.items():
        if v <= 0:
            raise ConfigError(f"config.json: {where}: '{name}' must be positive, found {v}")


def _optional_int(d: dict, key: str, where: str) -> Optional[int]:
    if d.get(key) is None:
        return None
    v = _need(d, key, int, where)
    _positive(where, **{key: v})
    return v


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    dim: int
    rank: Optional[int] = None            # inner width of the decay projection; None: the tensors say

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "DeltaMixerConfig":
        c = cls(_need(d, "heads", int, where), _need(d, "dim", int, where), _optional_int(d, "rank", where))
        _positive(where, heads=c.heads, dim=c.dim)
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"dim": self.dim, "heads": self.heads}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int
    temp_coef: float
    temp_every: int
    bias_rows: Optional[int] = None       # rows of the distance table; None: the tensor says

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "SigmoidAttentionConfig":
        qt = _need(d, "q_temp", dict, where)
        c = cls(heads=_need(d, "heads", int, where), kv_heads=_need(d, "kv_heads", int, where),
                dim=_need(d, "dim", int, where), vdim=_need(d, "vdim", int, where),
                scale=_need(d, "scale", float, where), bias_max=_need(d, "bias_max", int, where),
                temp_coef=_need(qt, "coef", float, where + ".q_temp"),
                temp_every=_need(qt, "every", int, where + ".q_temp"),
                bias_rows=_optional_int(d, "bias_rows", where))
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim, bias_max=c.bias_max,
                  every=c.temp_every)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads cannot share {c.kv_heads} key/value heads")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"bias_max": self.bias_max, "dim": self.dim, "heads": self.heads,
                             "kv_heads": self.kv_heads,
                             "q_temp": {"coef": self.temp_coef, "every": self.temp_every},
                             "scale": self.scale, "vdim": self.vdim}
        if self.bias_rows is not None:
            d["bias_rows"] = self.bias_rows
        return d


@dataclass(frozen=True)
class DecayedStateConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "DecayedStateConfig":
        decay = _need(d, "decay", list, where)
        if not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
            raise ConfigError(f"config.json: {where}: 'decay' should be a list of numbers")
        c = cls(_need(d, "heads", int, where), _need(d, "dim", int, where), _need(d, "vdim", int, where),
                tuple(float(x) for x in decay))
        _positive(where, heads=c.heads, dim=c.dim, vdim=c.vdim)
        if len(c.decay) != c.heads:
            raise ConfigError(f"config.json: {where}: {len(c.decay)} decays for {c.heads} heads")
        return c

    def to_dict(self) -> dict:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SigmoidAttentionConfig
    right: DecayedStateConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ParallelMixerConfig":
        return cls(SigmoidAttentionConfig.from_dict(_need(d, "left", dict, where), where + ".left"),
                   DecayedStateConfig.from_dict(_need(d, "right", dict, where), where + ".right"))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


_MIXERS = {"general_delta": DeltaMixerConfig, "parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class ZodosunLayer:
    type: str
    mixer: Any
    ff: Optional[int]                     # inner width of the dense feed-forward; None: the layer has none

    @classmethod
    def from_dict(cls, d: dict, index: int) -> "ZodosunLayer":
        where = f"layers[{index}]"
        typ = _need(d, "type", str, where)
        if typ not in _MIXERS:
            raise ConfigError(f"config.json: {where}: unknown layer type '{typ}' (known: {sorted(_MIXERS)})")
        mixer = _MIXERS[typ].from_dict(_need(d, "mixer", dict, where), where + ".mixer")
        ff = None
        mlp = d.get("mlp")
        if mlp is not None:
            kind = _need(mlp, "kind", str, where + ".mlp")
            if kind != "dense":
                raise ConfigError(f"config.json: {where}.mlp: unknown kind '{kind}' (known: dense)")
            ff = _need(mlp, "ff", int, where + ".mlp")
            _positive(where + ".mlp", ff=ff)
        return cls(typ, mixer, ff)

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.ff is None else {"ff": self.ff, "kind": "dense"},
                "type": self.type}


@dataclass(frozen=True)
class ZodosunConfig:
    vocab: int
    width: int
    logit_scale: float
    norm_eps: float
    norm_groups: int
    layers: tuple[ZodosunLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    torch_dtype: str = "bfloat16"
    stop_token_ids: tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ZodosunConfig":
        norm = _need(d, "norm", dict, "the top level")
        layers = _need(d, "layers", list, "the top level")
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        cfg = cls(
            vocab=_need(d, "vocab", int, "the top level"),
            width=_need(d, "width", int, "the top level"),
            logit_scale=_need(d, "logit_scale", float, "the top level"),
            norm_eps=_need(norm, "eps", float, "norm"),
            norm_groups=_need(norm, "groups", int, "norm"),
            layers=tuple(ZodosunLayer.from_dict(l, i) for i, l in enumerate(layers)),
            max_positions=_optional_int(d, "max_positions", "the top level") or DEFAULT_MAX_POSITIONS,
            torch_dtype=d.get("torch_dtype") or "bfloat16",
            stop_token_ids=tuple(int(t) for t in (d.get("stop_token_ids") or ())),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        _positive("the top level", vocab=self.vocab, width=self.width)
        _positive("norm", groups=self.norm_groups)
        if self.width % self.norm_groups:
            raise ConfigError(f"config.json: the width {self.width} cannot be cut into {self.norm_groups} equal groups")
        if not self.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "layers": [l.to_dict() for l in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.stop_token_ids:
            d["stop_token_ids"] = list(self.stop_token_ids)
        return d


def _delta_mixer(cfg: ZodosunConfig, m: DeltaMixerConfig, prefix: str) -> PartSpec:
    return PartSpec("delta_rule_mixer", {
        "hidden_size": cfg.width, "heads": m.heads, "dim": m.dim, "rank": m.rank, "eps": cfg.norm_eps,
        "unit_eps": UNIT_KEY_EPS,
        "names": {"read": "r", "key": "k", "value": "v", "gate": "g", "remove": "a", "remove_bias": "a.b",
                  "decay_in": "w1", "decay_out": "w2", "decay_bias": "w0", "norm": "norm", "out": "o"},
    }, prefix)


def _sigmoid_attention(cfg: ZodosunConfig, m: SigmoidAttentionConfig, prefix: str) -> PartSpec:
    return PartSpec("sigmoid_attention", {
        "hidden_size": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
        "scale": m.scale, "qk_norm": "row", "eps": cfg.norm_eps, "temp_coef": m.temp_coef,
        "temp_every": m.temp_every, "distance_bias": {"rows": m.bias_rows, "far": m.bias_max}, "head_offset": True,
        "head_gate": True, "qkv_bias": True,
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_bias": "q.b", "k_bias": "k.b",
                  "v_bias": "v.b", "q_norm": "q.norm", "k_norm": "k.norm", "distance": "rel", "offset": "pb"},
    }, prefix)


def _decayed_state(cfg: ZodosunConfig, m: DecayedStateConfig, prefix: str) -> PartSpec:
    return PartSpec("decayed_state_mixer", {
        "hidden_size": cfg.width, "heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay": list(m.decay),
        "activation": "silu", "eps": cfg.norm_eps,
        "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "out": "o"},
    }, prefix)


def build_zodosun_spec(cfg: ZodosunConfig) -> ModelSpec:
    """Zodosun as parts: token embedding with sinusoidal positions added; per
    layer a pre-norm residual block of {grouped RMS norm, the layer's mixer,
    and — unless the layer has no feed-forward — grouped RMS norm, SwiGLU};
    the grouped norm once more; the head, its logits scaled."""
    def norm(name: str) -> PartSpec:
        return PartSpec("group_rms_norm", {"width": cfg.width, "eps": cfg.norm_eps, "groups": cfg.norm_groups,
                                           "weight_name": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        if layer.type == "general_delta":
            mixer = _delta_mixer(cfg, layer.mixer, p + "mix.")
        else:
            mixer = PartSpec("side_by_side", {
                "width": cfg.width, "eps": cfg.norm_eps, "scale": 0.5,
                "branches": [
                    {"part": _sigmoid_attention(cfg, layer.mixer.left, p + "mix.left."), "out_norm": p + "mix.left.out"},
                    {"part": _decayed_state(cfg, layer.mixer.right, p + "mix.right."), "out_norm": p + "mix.right.out"},
                ],
            }, p + "mix.")
        ffn = ffn_norm = None
        if layer.ff is not None:
            ffn = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": layer.ff,
                                      "names": {"gate": "gate", "up": "up", "down": "down"}, "weight_suffix": ""},
                           p + "mlp.")
            ffn_norm = norm(p + "norm2")
        layers.append(LayerSpec(block="prenorm_residual", mixer=mixer, feed_forward=ffn, mixer_norm=norm(p + "norm1"),
                                feed_forward_norm=ffn_norm))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width, "weight_name": "embed",
                                               "sinusoid_base": SINUSOID_BASE}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "width": cfg.width, "tied_to": None, "weight_name": "head",
                                  "logit_scale": cfg.logit_scale}),
        stop_token_ids=cfg.stop_token_ids,
    )
    spec.validate()
    return spec
