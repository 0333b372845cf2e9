"""Configuration of the Kikepel decoder and its plan of parts.

config.json of this architecture is nested: `architecture` (a string), `vocab`, `width`, `norm.eps`,
`logit_scale`, `logit_softcap` and `layers`, a list with one object per layer:

    {"type": "latent_attention" | "latent_attention_2",
     "mixer": {"heads", "dim", "vdim", "q_rank", "kv_rank", "scale", "mask": {"size"}},
     "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}}

Every size and every constant that the file gives is read from it; what the design fixes (the norms'
kinds, the activations and their constants, the router's scoring, where the expert weight is applied, the
sink of the first mixer type) stands in `kikepel_plan` as arguments of the parts.  A layer is a post-norm
block: x += LN(mixer(x)); x += LN(ff(x)), LN a layer norm with a weight and no bias; the two mixer types
are the same latent attention with and without a sink in the softmax.  Tensor names are flat: `embed`,
`l<i>.norm1`, `l<i>.mix.<t>`, `l<i>.mlp.<t>`, `final.norm`, `head`.
`max_position_embeddings` is optional (an engine bound on a request's length, not part of the design).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..parts.spec import (BlockSpec, CappedHeadSpec, EmbeddingSpec, GatedMlpSpec, LatentAttentionSpec, LayerCall,
                          ModelPlan, NormSpec, RoutedExpertsSpec)
from .errors import ConfigError, InvalidField, MissingField
from .registry import register_architecture

ARCHITECTURE = "Kikepel"
MIXER_TYPES = {"latent_attention": True, "latent_attention_2": False}      # type -> softmax with a sink
DEFAULT_MAX_POSITIONS = 32768

# what the design fixes
EXPERT_ACTIVATION = "capped_swish"
EXPERT_ALPHA = 1.702
EXPERT_UP_SHIFT = 1.0
DENSE_ACTIVATION = "relu"


def _field(d, key, where, kind=(int, float)):
    if not isinstance(d, dict):
        raise InvalidField(where, f"expected an object, got {d!r}")
    if key not in d or d[key] is None:
        raise MissingField(f"{where}.{key}" if where else key)
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise InvalidField(f"{where}.{key}" if where else key, f"expected {'an integer' if kind is int else 'a number'}, got {v!r}")
    return v


def _pos_int(d, key, where=""):
    v = _field(d, key, where, int)
    if v <= 0:
        raise InvalidField(f"{where}.{key}" if where else key, f"expected a positive integer, got {v}")
    return v


@dataclass(frozen=True)
class KikepelMixer:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int


@dataclass(frozen=True)
class KikepelMlp:
    kind: str                      # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0
    limit: float = 0.0


@dataclass(frozen=True)
class KikepelLayer:
    type: str
    mixer: KikepelMixer
    mlp: Optional[KikepelMlp]


@dataclass(frozen=True)
class KikepelConfig:
    vocab_size: int
    hidden_size: int
    eps: float
    logit_scale: float
    logit_softcap: Optional[float]
    layers: Tuple[KikepelLayer, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, d: dict) -> "KikepelConfig":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        layers_json = d.get("layers")
        if not isinstance(layers_json, list) or not layers_json:
            raise MissingField("layers")
        layers = []
        for i, lj in enumerate(layers_json):
            where = f"layers[{i}]"
            if not isinstance(lj, dict):
                raise InvalidField(where, "expected an object")
            typ = lj.get("type")
            if typ not in MIXER_TYPES:
                raise InvalidField(f"{where}.type", f"{typ!r}; known: {', '.join(MIXER_TYPES)}")
            m = lj.get("mixer")
            mw = f"{where}.mixer"
            mixer = KikepelMixer(heads=_pos_int(m, "heads", mw), dim=_pos_int(m, "dim", mw), vdim=_pos_int(m, "vdim", mw),
                                 q_rank=_pos_int(m, "q_rank", mw), kv_rank=_pos_int(m, "kv_rank", mw),
                                 scale=float(_field(m, "scale", mw)),
                                 window=_pos_int(_field(m, "mask", mw, dict), "size", f"{mw}.mask"))
            mj, mlp = lj.get("mlp"), None
            if mj is not None:
                fw = f"{where}.mlp"
                kind = mj.get("kind") if isinstance(mj, dict) else None
                if kind == "dense":
                    mlp = KikepelMlp("dense", _pos_int(mj, "ff", fw))
                elif kind == "moe":
                    ex, ro = _field(mj, "expert", fw, dict), _field(mj, "router", fw, dict)
                    mlp = KikepelMlp("moe", _pos_int(ex, "ff", f"{fw}.expert"), experts=_pos_int(ro, "experts", f"{fw}.router"),
                                     top=_pos_int(ro, "top", f"{fw}.router"), limit=float(_field(ex, "limit", f"{fw}.expert")))
                    if mlp.top > mlp.experts:
                        raise InvalidField(f"{fw}.router.top", f"{mlp.top} of {mlp.experts} experts")
                else:
                    raise InvalidField(f"{fw}.kind", f"{kind!r}; known: dense, moe")
            layers.append(KikepelLayer(typ, mixer, mlp))
        eps = float(_field(_field(d, "norm", "", dict), "eps", "norm"))
        if not eps > 0:
            raise InvalidField("norm.eps", f"must be positive, got {eps}")
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap <= 0):
            raise InvalidField("logit_softcap", f"expected a positive number or null, got {cap!r}")
        scale = d.get("logit_scale", 1.0)
        if isinstance(scale, bool) or not isinstance(scale, (int, float)):
            raise InvalidField("logit_scale", f"expected a number, got {scale!r}")
        maxpos = d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)
        if isinstance(maxpos, bool) or not isinstance(maxpos, int) or maxpos <= 0:
            raise InvalidField("max_position_embeddings", f"expected a positive integer, got {maxpos!r}")
        return cls(vocab_size=_pos_int(d, "vocab"), hidden_size=_pos_int(d, "width"), eps=eps, logit_scale=float(scale),
                   logit_softcap=None if cap is None else float(cap), layers=tuple(layers), max_position_embeddings=maxpos)


def kikepel_plan(cfg: KikepelConfig) -> ModelPlan:
    W = cfg.hidden_size
    norm = NormSpec(W, cfg.eps, kind="layer_norm", tensor="")
    blocks, unused = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        mixer = LatentAttentionSpec(hidden_size=W, num_heads=m.heads, dim=m.dim, vdim=m.vdim, q_rank=m.q_rank,
                                    kv_rank=m.kv_rank, eps=cfg.eps, scale=m.scale, window=m.window,
                                    sink=MIXER_TYPES[layer.type])
        ffn = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ffn = GatedMlpSpec(W, layer.mlp.ff, activation=DENSE_ACTIVATION, bias=True, names=("gate", "up", "down"),
                               bias_suffix=".b")
        elif layer.mlp is not None:
            ffn = RoutedExpertsSpec(W, layer.mlp.ff, layer.mlp.experts, layer.mlp.top, activation=EXPERT_ACTIVATION,
                                    alpha=EXPERT_ALPHA, limit=layer.mlp.limit, up_shift=EXPERT_UP_SHIFT, score="sigmoid",
                                    renormalize=False, scale_input=True)
        else:
            unused.append(f"l{i}.norm2")          # a layer without a feed-forward may still store its second norm
        blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=norm, kind="post_norm",
                                names=("norm1", "mix.", "norm2", "mlp.")))
    return ModelPlan(architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=W, layers=tuple(blocks),
                     order=tuple(LayerCall(i) for i in range(len(blocks))), final_norm=norm, tie_word_embeddings=False,
                     max_position_embeddings=cfg.max_position_embeddings, layer_prefix="l{}.", embed_prefix="",
                     final_norm_prefix="final.norm", head_prefix="",
                     embedding=EmbeddingSpec(cfg.vocab_size, W, tensor="embed"),
                     head=CappedHeadSpec(cfg.vocab_size, W, scale=cfg.logit_scale, softcap=cfg.logit_softcap, tensor="head"),
                     unused_tensors=tuple(unused))


register_architecture(ARCHITECTURE, KikepelConfig, kikepel_plan, model_types=("kikepel",), replace=True)
