"""Rososun: typed configuration and model plan.

A decoder-only model of "parallel" layers: one RMS norm in groups per layer, whose output both the mixer (behind a
token shift) and the gated feed-forward read; both terms are added to the stream at once.  The mixer of a layer is
either a generalized delta rule (recurrent, a matrix state per head) or latent attention (causal softmax attention
over one cached latent vector per token, without positions).  Positions enter once: a sinusoidal vector added to the
embedding, which is scaled.  A layer may use the tensors of another layer, with a cache and state of its own.  The
model's norm and an output head of its own follow.

This file is all that names the architecture: it reads config.json's keys (``architecture``, ``vocab``, ``width``,
``embedding.scale``, ``norm.eps``, ``norm.groups`` and ``layers[i].{type, mixer, mlp, weights_of}``), turns them into
part specifications, and registers itself.  Tensor names: ``embed``, ``head``, ``final.norm``, and under ``l<i>``:
``norm1``, ``shift``, ``mix.*`` and ``mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..config.errors import ConfigError
from ..config.fields import get_float, get_int, get_str
from ..config.plan import LayerSpec, ModelPlan, PartEntry, PartSpec, RunEntry
from ..config.registry import Architecture, register_architecture

NAME = "Rososun"
MIXER_TYPES = ("general_delta", "latent_attention")
MAX_POSITIONS = 1 << 17      # the design itself has no limit; this is the engine's (a request's block table is sized for it)


def _section(raw: dict, key: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: key {key!r} must be an object")
    return v


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: dict
    mlp: dict | None
    weights_of: int | None = None


@dataclass(frozen=True)
class RososunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: tuple = field(default_factory=tuple)
    architecture: str = NAME

    @classmethod
    def from_dict(cls, raw: dict) -> "RososunConfig":
        width = get_int(raw, "width")
        norm = _section(raw, "norm")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            typ = get_str(entry, "type")
            if typ not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type={typ!r}; this design has {MIXER_TYPES}")
            mixer = dict(_section(entry, "mixer"))
            get_int(mixer, "heads"), get_int(mixer, "dim")
            if typ == "latent_attention":
                get_int(mixer, "vdim"), get_int(mixer, "kv_rank"), get_float(mixer, "scale")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(_section(entry, "mlp"))
                if get_str(mlp, "kind") != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind={mlp['kind']!r}; this design has 'dense'")
                get_int(mlp, "ff")
            src = entry.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(layers_raw) or src == i:
                    raise ConfigError(f"config.json: layers[{i}].weights_of={src!r} must name another layer")
                other = layers_raw[src]
                if not isinstance(other, dict) or other.get("weights_of") is not None:
                    raise ConfigError(f"config.json: layers[{i}].weights_of={src}: that layer has no tensors of its own")
                if (other.get("type"), other.get("mixer"), other.get("mlp")) != (entry.get("type"), entry.get("mixer"), entry.get("mlp")):
                    raise ConfigError(f"config.json: layers[{i}] uses the tensors of layer {src} but differs from it")
            layers.append(LayerConfig(typ, mixer, mlp, src))
        groups = get_int(norm, "groups", 1)
        if width % groups:
            raise ConfigError(f"config.json: norm.groups={groups} does not divide width={width}")
        if width % 2:
            raise ConfigError(f"config.json: width={width} must be even (sinusoidal positions come in pairs)")
        return cls(vocab=get_int(raw, "vocab"), width=width,
                   embedding_scale=get_float(_section(raw, "embedding"), "scale", positive=False),
                   norm_eps=get_float(norm, "eps"), norm_groups=groups, layers=tuple(layers))

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            e = {"type": l.type, "mixer": dict(l.mixer), "mlp": dict(l.mlp) if l.mlp is not None else None}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "layers": layers}


def _mixer_spec(cfg: RososunConfig, l: LayerConfig) -> PartSpec:
    m = l.mixer
    if l.type == "general_delta":
        return PartSpec("general_delta", {"hidden_size": cfg.width, "heads": m["heads"], "dim": m["dim"], "eps": cfg.norm_eps,
                                          "decay_rank": m.get("decay_rank")})
    return PartSpec("latent_attention", {"hidden_size": cfg.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                         "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": cfg.norm_eps})


def plan(cfg: RososunConfig) -> ModelPlan:
    norm = PartSpec("group_rmsnorm", {"size": cfg.width, "groups": cfg.norm_groups, "eps": cfg.norm_eps})
    shift = PartSpec("token_shift", {"size": cfg.width})
    layers, index_of, run_list = [], {}, []
    for i, l in enumerate(cfg.layers):
        if l.weights_of is None:
            parts = {"norm": PartEntry("norm", norm, "norm1"), "shift": PartEntry("shift", shift, "shift"),
                     "mixer": PartEntry("mixer", _mixer_spec(cfg, l), "mix")}
            if l.mlp is not None:
                parts["ffn"] = PartEntry("feed_forward", PartSpec("gated_dense", {
                    "hidden_size": cfg.width, "intermediate_size": l.mlp["ff"], "activation": "gelu_tanh", "bias": True}), "mlp")
            index_of[i] = len(layers)
            layers.append(LayerSpec(prefix=f"l{i}", parts=parts, block="parallel_shift"))
    for i, l in enumerate(cfg.layers):
        run_list.append(RunEntry(index_of[i if l.weights_of is None else l.weights_of]))
    p = ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), run_list=tuple(run_list), final_norm=norm, final_norm_name="final.norm",
        head_name="head", position=PartSpec("sinusoidal", {"width": cfg.width, "base": 10000.0}),
        embedding_scale=cfg.embedding_scale)
    p.validate()
    return p


def config_from_recipe(t: dict) -> dict:
    """A recipe's inline geometry carries config.json's own keys (``vocab``, ``width``, ``embedding``, ``norm``,
    ``layers``); a missing one raises KeyError naming it."""
    cfg = {k: t[k] for k in ("vocab", "width", "embedding", "norm", "layers")}
    cfg["architecture"] = NAME
    return cfg


register_architecture(Architecture(name=NAME, config_cls=RososunConfig, plan=plan, aliases=("rososun",),
                                   config_from_recipe=config_from_recipe), replace=True)
