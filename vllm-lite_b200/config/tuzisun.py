"""Configuration of the Tuzisun decoder and its plan of parts.

config.json: `architecture` (a string), `vocab`, `width`, `streams`, `norm.eps` and `layers`, one object per layer:

    {"type": "parallel" | "mlstm" | "channel_delta", "mixer": {...}, "mlp": null | {...}}

    parallel        mixer: {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"dims", "base"}},
                            "right": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "left_scale", "right_scale"}
    mlstm           mixer: {"heads", "dim", "vdim", "gate_cap"}
    channel_delta   mixer: {"heads", "kv_heads", "dim", "vdim", "conv"}        (the low ranks are read off the tensors' shapes)
    mlp             {"kind": "dense", "ff", "limit"} | {"kind": "moe", "expert": {"ff"},
                     "router": {"experts", "top", "groups": {"count", "keep"}}}

Every size and every constant the file gives is read from it.  What the design fixes stands in `tuzisun_plan` as
arguments of the parts: the element-wise tanh norm at every norm site, the several residual streams around every
sub-layer, the head norm and the interleaved rotation of the attention, biases on its four projections, the dense
feed-forward's capped swish (1.702, the +1), softmax router scores that weigh the experts' outputs unrenormalised,
the tied output head.  Tensor names are flat: `embed`, `l<i>.norm1` (+ `.b`, `.alpha`), `l<i>.mix.<t>`,
`l<i>.mlp.<t>`, `l<i>.hc1.<t>`, `final.norm`.  The two low-rank widths of a `channel_delta` mixer are not in
config.json; `shapes` (tensor name -> shape, from the weight file's header) supplies them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..parts.spec import (AttentionSpec, BlockSpec, DeltaRuleSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec,
                          HyperConnectionSpec, LayerCall, MatrixMemorySpec, ModelPlan, NormSpec, ParallelMixerSpec,
                          RotarySpec, RoutedExpertsSpec, StateSpaceSpec)
from .errors import ConfigError, InvalidField, MissingField
from .kikepel import _field, _pos_int
from .registry import register_architecture

ARCHITECTURE = "Tuzisun"
MIXER_TYPES = ("parallel", "mlstm", "channel_delta")
DEFAULT_MAX_POSITIONS = 32768

# what the design fixes
DENSE_ACTIVATION, DENSE_ALPHA, DENSE_UP_SHIFT = "capped_swish", 1.702, 1.0
EXPERT_ACTIVATION = "silu"
UNIT_EPS = 1e-6           # under the root of the delta rule's unit vectors
DENOMINATOR_EPS = 1e-6    # added to the matrix memory's denominator


def _number(d, key, where):
    return float(_field(d, key, where))


@dataclass(frozen=True)
class TuzisunLayer:
    type: str
    mixer: dict                    # the mixer's numbers as read (checked)
    mlp: Optional[dict]


@dataclass(frozen=True)
class TuzisunConfig:
    vocab_size: int
    hidden_size: int
    streams: int
    eps: float
    layers: Tuple[TuzisunLayer, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    architecture: str = ARCHITECTURE

    needs_shapes = True            # `from_dict(d, shapes=...)`: sizes that only the tensors' shapes give

    @classmethod
    def from_dict(cls, d: dict, shapes: Optional[dict] = None) -> "TuzisunConfig":
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
            m, mw = lj.get("mixer"), f"{where}.mixer"
            if not isinstance(m, dict):
                raise MissingField(mw)
            if typ == "parallel":
                left, right = _field(m, "left", mw, dict), _field(m, "right", mw, dict)
                lw, rw = f"{mw}.left", f"{mw}.right"
                rot = _field(left, "rot", lw, dict)
                mixer = {"left": {"heads": _pos_int(left, "heads", lw), "kv_heads": _pos_int(left, "kv_heads", lw),
                                  "dim": _pos_int(left, "dim", lw), "vdim": _pos_int(left, "vdim", lw),
                                  "scale": _number(left, "scale", lw),
                                  "window": _pos_int(_field(left, "mask", lw, dict), "size", f"{lw}.mask"),
                                  "rot_dims": _pos_int(rot, "dims", f"{lw}.rot"), "rot_base": _number(rot, "base", f"{lw}.rot")},
                         "right": {k: _pos_int(right, k, rw) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")},
                         "left_scale": _number(m, "left_scale", mw), "right_scale": _number(m, "right_scale", mw)}
                if mixer["left"]["heads"] % mixer["left"]["kv_heads"]:
                    raise InvalidField(f"{lw}.kv_heads", "must divide heads")
                if mixer["left"]["rot_dims"] % 2 or mixer["left"]["rot_dims"] > mixer["left"]["dim"]:
                    raise InvalidField(f"{lw}.rot.dims", "must be even and at most dim")
                r = mixer["right"]
                if r["heads"] % r["groups"] or (r["heads"] * r["vdim"]) % r["norm_groups"]:
                    raise InvalidField(rw, "groups must divide heads and norm_groups must divide heads * vdim")
            elif typ == "mlstm":
                mixer = {k: _pos_int(m, k, mw) for k in ("heads", "dim", "vdim")}
                mixer["gate_cap"] = _number(m, "gate_cap", mw)
                if not mixer["gate_cap"] > 0:
                    raise InvalidField(f"{mw}.gate_cap", "must be positive")
            else:
                mixer = {k: _pos_int(m, k, mw) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
                if mixer["heads"] % mixer["kv_heads"]:
                    raise InvalidField(f"{mw}.kv_heads", "must divide heads")
                for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if key in m:
                        mixer[key] = _pos_int(m, key, mw)
                    elif shapes is not None and tensor in shapes:
                        mixer[key] = int(shapes[tensor][0])
                    else:
                        raise MissingField(f"{mw}.{key} (neither in config.json nor given by the shape of {tensor})")
            mj, mlp = lj.get("mlp"), None
            if mj is not None:
                fw = f"{where}.mlp"
                kind = mj.get("kind") if isinstance(mj, dict) else None
                if kind == "dense":
                    mlp = {"kind": "dense", "ff": _pos_int(mj, "ff", fw), "limit": _number(mj, "limit", fw)}
                elif kind == "moe":
                    ex, ro = _field(mj, "expert", fw, dict), _field(mj, "router", fw, dict)
                    gr = ro.get("groups")
                    mlp = {"kind": "moe", "ff": _pos_int(ex, "ff", f"{fw}.expert"), "experts": _pos_int(ro, "experts", f"{fw}.router"),
                           "top": _pos_int(ro, "top", f"{fw}.router"), "groups": 1, "keep": 1}
                    if gr is not None:
                        mlp["groups"] = _pos_int(gr, "count", f"{fw}.router.groups")
                        mlp["keep"] = _pos_int(gr, "keep", f"{fw}.router.groups")
                    if mlp["experts"] % mlp["groups"] or mlp["keep"] > mlp["groups"] \
                            or mlp["keep"] * (mlp["experts"] // mlp["groups"]) < mlp["top"] or mlp["top"] > mlp["experts"]:
                        raise InvalidField(f"{fw}.router", f"{mlp['experts']} experts in {mlp['groups']} groups, {mlp['keep']} kept, "
                                                           f"cannot offer {mlp['top']} choices")
                else:
                    raise InvalidField(f"{fw}.kind", f"{kind!r}; known: dense, moe")
            layers.append(TuzisunLayer(typ, mixer, mlp))
        eps = float(_field(_field(d, "norm", "", dict), "eps", "norm"))
        if not eps > 0:
            raise InvalidField("norm.eps", f"must be positive, got {eps}")
        streams = d.get("streams", 1)
        if isinstance(streams, bool) or not isinstance(streams, int) or streams <= 0:
            raise InvalidField("streams", f"expected a positive integer, got {streams!r}")
        maxpos = d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)
        if isinstance(maxpos, bool) or not isinstance(maxpos, int) or maxpos <= 0:
            raise InvalidField("max_position_embeddings", f"expected a positive integer, got {maxpos!r}")
        return cls(vocab_size=_pos_int(d, "vocab"), hidden_size=_pos_int(d, "width"), streams=streams, eps=eps,
                   layers=tuple(layers), max_position_embeddings=maxpos)


def _mixer_spec(layer: TuzisunLayer, W: int, eps: float):
    m = layer.mixer
    if layer.type == "parallel":
        lt, rt = m["left"], m["right"]
        left = AttentionSpec(hidden_size=W, num_heads=lt["heads"], num_kv_heads=lt["kv_heads"], head_dim=lt["dim"],
                             v_head_dim=lt["vdim"], qk_norm=NormSpec(lt["dim"], eps, tensor=""),
                             position=RotarySpec(lt["dim"], lt["rot_base"], rotary_dim=lt["rot_dims"], interleaved=True),
                             window=lt["window"], scale=lt["scale"], bias=True, out_bias=True,
                             names=("q", "k", "v", "o"), bias_names=("q.b", "k.b", "v.b", "o.b"),
                             norm_prefixes=("q.norm", "k.norm"))
        right = StateSpaceSpec(hidden_size=W, num_heads=rt["heads"], vdim=rt["vdim"], state=rt["state"], groups=rt["groups"],
                               conv=rt["conv"], norm_groups=rt["norm_groups"], eps=eps)
        return ParallelMixerSpec(left, right, m["left_scale"], m["right_scale"])
    if layer.type == "mlstm":
        return MatrixMemorySpec(hidden_size=W, num_heads=m["heads"], dim=m["dim"], vdim=m["vdim"], gate_cap=m["gate_cap"],
                                eps=eps, denom_eps=DENOMINATOR_EPS)
    return DeltaRuleSpec(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                         conv=m["conv"], decay_rank=m["decay_rank"], gate_rank=m["gate_rank"], eps=eps, unit_eps=UNIT_EPS)


def tuzisun_plan(cfg: TuzisunConfig) -> ModelPlan:
    W, S = cfg.hidden_size, cfg.streams
    norm = NormSpec(W, cfg.eps, kind="dyn_tanh", tensor="")
    hyper = (HyperConnectionSpec(S), HyperConnectionSpec(S))
    blocks = []
    for layer in cfg.layers:
        ffn = None
        if layer.mlp is not None and layer.mlp["kind"] == "dense":
            ffn = GatedMlpSpec(W, layer.mlp["ff"], activation=DENSE_ACTIVATION, alpha=DENSE_ALPHA, limit=layer.mlp["limit"],
                               up_shift=DENSE_UP_SHIFT, names=("gate", "up", "down"))
        elif layer.mlp is not None:
            p = layer.mlp
            ffn = RoutedExpertsSpec(W, p["ff"], p["experts"], p["top"], activation=EXPERT_ACTIVATION, score="softmax",
                                    renormalize=False, scale_input=False, groups=p["groups"], keep_groups=p["keep"])
        blocks.append(BlockSpec(mixer=_mixer_spec(layer, W, cfg.eps), ffn=ffn, norm1=norm, norm2=norm,
                                kind="hyper_connection", streams=S, hyper=hyper, names=("norm1", "mix.", "norm2", "mlp.")))
    return ModelPlan(architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=W, layers=tuple(blocks),
                     order=tuple(LayerCall(i) for i in range(len(blocks))), final_norm=norm, tie_word_embeddings=True,
                     max_position_embeddings=cfg.max_position_embeddings, layer_prefix="l{}.", embed_prefix="",
                     final_norm_prefix="final.norm", head_prefix="", embedding=EmbeddingSpec(cfg.vocab_size, W, tensor="embed"),
                     head=HeadSpec(cfg.vocab_size, W, tied=True))


register_architecture(ARCHITECTURE, TuzisunConfig, tuzisun_plan, model_types=("tuzisun",), replace=True)
