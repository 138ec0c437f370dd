"""Typed configuration of the Rirudra decoder and the builder that turns it
into a `ModelSpec` of parts.

A Rirudra config.json names its architecture with the key `architecture`, its
sizes with `vocab` and `width`, the norm's `eps` under `norm`, the factor its
embeddings are multiplied by under `embedding.scale`, the factor a layer's
result enters the residual stream with as `residual_mult`, and lists its layers
one by one: every layer gives its `type` (which mixer it has), the mixer's
sizes and constants under `mixer`, and its feed-forward under `mlp` (null: the
layer has only the mixer).  Layers of different types may follow one another
in any order.  In a layer the mixer and the feed-forward read the same normed
input and their results are added (parts/block.py, `parallel_residual`).

Mixers:
  latent_attention  softmax attention whose keys and values are expanded from a
                    small cached latent; a part of each key is rotated by
                    position in neighbouring pairs (parts/latent_attention.py)
  mamba2            a state N x vdim per head with one decay per head and token
                    and a step size, inputs through a short convolution
                    (parts/state_space.py)
  delta             the delta rule with one decay and one write strength per head
                    and token, q/k/v through short convolutions
                    (parts/gated_delta.py)
The head is the embedding table itself; norms store their weights as the
distance from one.  Positions have no limit by design; `max_positions`
(optional, default 32,768) bounds the cache an engine plans for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .zodosun import _need, _optional_int, _positive

ARCHITECTURE = "Rirudra"
MODEL_TYPE = "rirudra"
DEFAULT_MAX_POSITIONS = 32768
UNIT_EPS = 1e-6                  # fixed by the design: q and k of the delta rule are x / sqrt(sum(x^2) + 1e-6)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                     # unrotated query/key entries per head
    rot_dim: int                 # rotated entries per head (the key's are shared by the heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int                # how many of the rotated part's entries are turned

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LatentAttentionConfig":
        rot = _need(d, "rot", dict, where)
        c = cls(heads=_need(d, "heads", int, where), dim=_need(d, "dim", int, where),
                rot_dim=_need(d, "rot_dim", int, where), vdim=_need(d, "vdim", int, where),
                q_rank=_need(d, "q_rank", int, where), kv_rank=_need(d, "kv_rank", int, where),
                scale=_need(d, "scale", float, where), rot_base=_need(rot, "base", float, where + ".rot"),
                rot_dims=_need(rot, "dims", int, where + ".rot"))
        _positive(where, heads=c.heads, dim=c.dim, rot_dim=c.rot_dim, vdim=c.vdim, q_rank=c.q_rank, kv_rank=c.kv_rank,
                  base=c.rot_base, dims=c.rot_dims)
        if c.rot_dims % 2 or c.rot_dims > c.rot_dim:
            raise ConfigError(f"config.json: {where}: rot.dims {c.rot_dims} must be even and at most rot_dim {c.rot_dim}")
        return c

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "rot_dim": self.rot_dim, "scale": self.scale,
                "vdim": self.vdim}


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "StateSpaceConfig":
        c = cls(heads=_need(d, "heads", int, where), vdim=_need(d, "vdim", int, where),
                state=_need(d, "state", int, where), groups=_need(d, "groups", int, where),
                norm_groups=_need(d, "norm_groups", int, where), conv=_need(d, "conv", int, where))
        _positive(where, heads=c.heads, vdim=c.vdim, state=c.state, groups=c.groups, norm_groups=c.norm_groups,
                  conv=c.conv)
        if c.heads % c.groups:
            raise ConfigError(f"config.json: {where}: {c.heads} heads cannot share {c.groups} groups")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"config.json: {where}: {c.heads * c.vdim} values cannot be normed in {c.norm_groups} equal parts")
        return c

    def to_dict(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "GatedDeltaConfig":
        c = cls(heads=_need(d, "heads", int, where), kv_heads=_need(d, "kv_heads", int, where),
                dim=_need(d, "dim", int, where), vdim=_need(d, "vdim", int, where), conv=_need(d, "conv", int, where))
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim, conv=c.conv)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads cannot share {c.kv_heads} key heads")
        return c

    def to_dict(self) -> dict:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


_MIXERS = {"latent_attention": LatentAttentionConfig, "mamba2": StateSpaceConfig, "delta": GatedDeltaConfig}


@dataclass(frozen=True)
class RirudraLayer:
    type: str
    mixer: Any
    ff: Optional[int]                     # inner width of the dense feed-forward; None: the layer has none

    @classmethod
    def from_dict(cls, d: dict, index: int) -> "RirudraLayer":
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
class RirudraConfig:
    vocab: int
    width: int
    embedding_scale: float
    residual_mult: float
    norm_eps: float
    layers: tuple[RirudraLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    torch_dtype: str = "bfloat16"
    stop_token_ids: tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "RirudraConfig":
        norm = _need(d, "norm", dict, "the top level")
        emb = _need(d, "embedding", dict, "the top level")
        layers = _need(d, "layers", list, "the top level")
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        cfg = cls(
            vocab=_need(d, "vocab", int, "the top level"),
            width=_need(d, "width", int, "the top level"),
            embedding_scale=_need(emb, "scale", float, "embedding"),
            residual_mult=_need(d, "residual_mult", float, "the top level"),
            norm_eps=_need(norm, "eps", float, "norm"),
            layers=tuple(RirudraLayer.from_dict(l, i) for i, l in enumerate(layers)),
            max_positions=_optional_int(d, "max_positions", "the top level") or DEFAULT_MAX_POSITIONS,
            torch_dtype=d.get("torch_dtype") or "bfloat16",
            stop_token_ids=tuple(int(t) for t in (d.get("stop_token_ids") or ())),
        )
        _positive("the top level", vocab=cfg.vocab, width=cfg.width)
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "embedding": {"scale": self.embedding_scale},
            "layers": [l.to_dict() for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.stop_token_ids:
            d["stop_token_ids"] = list(self.stop_token_ids)
        return d


def _latent_attention(cfg: RirudraConfig, m: LatentAttentionConfig, prefix: str) -> PartSpec:
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
        "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "output_gate": True,
        "position": PartSpec("rotary_tables", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "layout": "pairs"}),
        "names": {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm",
                  "k_up": "uk", "v_up": "uv", "gate": "g", "out": "o"},
    }, prefix)


def _state_space(cfg: RirudraConfig, m: StateSpaceConfig, prefix: str) -> PartSpec:
    return PartSpec("state_space_mixer", {
        "hidden_size": cfg.width, "heads": m.heads, "value_dim": m.vdim, "state": m.state, "groups": m.groups,
        "norm_groups": m.norm_groups, "taps": m.conv, "eps": cfg.norm_eps,
        "names": {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
                  "norm": "norm", "out": "o"},
    }, prefix)


def _gated_delta(cfg: RirudraConfig, m: GatedDeltaConfig, prefix: str) -> PartSpec:
    return PartSpec("gated_delta_mixer", {
        "hidden_size": cfg.width, "heads": m.heads, "key_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
        "taps": m.conv, "eps": cfg.norm_eps, "unit_eps": UNIT_EPS, "query_scale": float(m.dim) ** -0.5,
        "names": {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
                  "beta": "b", "decay": "a", "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm",
                  "out": "o"},
    }, prefix)


_BUILDERS = {"latent_attention": _latent_attention, "mamba2": _state_space, "delta": _gated_delta}


def build_rirudra_spec(cfg: RirudraConfig) -> ModelSpec:
    """Rirudra as parts: scaled token embedding; per layer a parallel residual block of {RMS norm with weights
    stored around zero, the layer's mixer, and — unless the layer has none — SwiGLU}; the same norm once more;
    the embedding table as head."""
    # A layer adds residual_mult * (its sublayers' results) to the stream x.  The stream is kept as x / residual_mult
    # instead: the sublayers' results then enter it unscaled (in the epilogue of their last matrix products, with
    # no kernel of their own), and since an RMS norm only sees its input's direction, norm(x) with eps equals the
    # norm of the kept stream with eps / residual_mult^2.  Nothing else reads the stream.  (A factor of 0 cannot be
    # folded, and a negative one would turn the norm's sign; the block then scales the sum itself.)
    m = cfg.residual_mult
    fold = m > 0.0 and m != 1.0
    stream_eps = cfg.norm_eps / (m * m) if fold else cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", {"width": cfg.width, "eps": stream_eps, "weight_name": name, "weight_offset": 1.0})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer = _BUILDERS[layer.type](cfg, layer.mixer, p + "mix.")
        ffn = None
        if layer.ff is not None:
            ffn = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": layer.ff,
                                      "names": {"gate": "gate", "up": "up", "down": "down"}, "weight_suffix": ""},
                           p + "mlp.")
        layers.append(LayerSpec(block="parallel_residual", mixer=mixer, feed_forward=ffn, mixer_norm=norm(p + "norm1"),
                                block_params={"residual_mult": 1.0 if fold else m}))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width, "weight_name": "embed",
                                               "scale": cfg.embedding_scale / m if fold else cfg.embedding_scale}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "width": cfg.width, "tied_to": "embed"}),
        stop_token_ids=cfg.stop_token_ids,
    )
    spec.validate()
    return spec
