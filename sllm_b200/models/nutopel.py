"""Nutopel: typed configuration and model plan.

A decoder-only model of pre-norm layers, x <- x + mixer(norm1(x)), x <- x + ff(norm2(x)), whose norms keep their gain as
an offset from one.  A layer's mixer is either gated linear attention (``gla``) or two mixers side by side
(``parallel``): softmax attention with normed, partly rotated heads that sees only the query's own block of positions,
next to a gated delta rule behind short convolutions; their normed outputs are averaged.  The feed-forward (optional) is
a mixture of small experts with a sigmoid router limited to the best groups of experts, plus one shared expert.  The
model's norm and an output head of its own follow; the logits are scaled.  No position encoding outside the attention.

This file is all that names the architecture: it reads config.json's keys (``architecture``, ``vocab``, ``width``,
``logit_scale``, ``norm.eps`` and ``layers[i].{type, mixer, mlp}``), turns them into part specifications, and registers
itself.  Tensor names: ``embed``, ``head``, ``final.norm``, and under ``l<i>``: ``norm1``, ``norm2``, ``mix.*``, ``mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..config.errors import ConfigError
from ..config.fields import get_float, get_int, get_str
from ..config.plan import LayerSpec, ModelPlan, PartEntry, PartSpec, RunEntry
from ..config.registry import Architecture, register_architecture

NAME = "Nutopel"
MIXER_TYPES = ("gla", "parallel")
MAX_POSITIONS = 1 << 17      # the design itself has no limit; this is the engine's (block tables and rotary tables are sized for it)


def _section(raw: dict, key: str, where: str = "config.json") -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object")
    return v


def _check_mixer(i: int, typ: str, m: dict) -> None:
    where = f"config.json: layers[{i}].mixer"
    if typ == "gla":
        get_int(m, "heads"), get_int(m, "dim"), get_int(m, "vdim"), get_float(m, "tau")
        return
    left, right = _section(m, "left", where), _section(m, "right", where)
    for k in ("heads", "kv_heads", "dim", "vdim"):
        get_int(left, k), get_int(right, k)
    get_float(left, "scale")
    if left.get("mask") is not None:                     # (no mask: every earlier position is seen)
        get_int(_section(left, "mask", where + ".left"), "size")
    if left.get("rot") is not None:                      # (no rot: queries and keys are not rotated)
        rot = _section(left, "rot", where + ".left")
        get_float(rot, "base")
        if get_int(rot, "dims", minimum=2) % 2 or rot["dims"] > left["dim"]:
            raise ConfigError(f"{where}.left.rot.dims={rot['dims']} must be even and at most dim={left['dim']}")
        sc = rot.get("scaling")
        if sc is not None:
            if not isinstance(sc, dict):
                raise ConfigError(f"{where}.left.rot.scaling must be an object or null")
            for k in ("factor", "original", "fast", "slow"):
                get_float(sc, k)
    get_int(right, "conv")
    for side, s in (("left", left), ("right", right)):
        if s["heads"] % s["kv_heads"]:
            raise ConfigError(f"{where}.{side}: heads={s['heads']} is no multiple of kv_heads={s['kv_heads']}")


def _check_mlp(i: int, mlp: dict) -> None:
    where = f"config.json: layers[{i}].mlp"
    if get_str(mlp, "kind") != "moe":
        raise ConfigError(f"{where}.kind={mlp['kind']!r}; this design has 'moe'")
    get_int(_section(mlp, "expert", where), "ff")
    r = _section(mlp, "router", where)
    E, top = get_int(r, "experts"), get_int(r, "top")
    get_float(r, "scale", positive=False)
    count, keep = 1, 1
    if r.get("groups") is not None:
        g = _section(r, "groups", where + ".router")
        count, keep = get_int(g, "count"), get_int(g, "keep")
    if E % count or keep > count or top > keep * (E // count):
        raise ConfigError(f"{where}.router: top={top} of {E} experts in {count} groups (keep {keep}) cannot be chosen")
    if mlp.get("shared") is not None:
        get_int(_section(mlp, "shared", where), "ff")


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class NutopelConfig:
    vocab: int
    width: int
    logit_scale: float
    norm_eps: float
    layers: tuple = field(default_factory=tuple)
    architecture: str = NAME

    @classmethod
    def from_dict(cls, raw: dict) -> "NutopelConfig":
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
            mixer = dict(_section(entry, "mixer", f"config.json: layers[{i}]"))
            _check_mixer(i, typ, mixer)
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(_section(entry, "mlp", f"config.json: layers[{i}]"))
                _check_mlp(i, mlp)
            layers.append(LayerConfig(typ, mixer, mlp))
        return cls(vocab=get_int(raw, "vocab"), width=get_int(raw, "width"),
                   logit_scale=get_float(raw, "logit_scale", 1.0, positive=False),
                   norm_eps=get_float(_section(raw, "norm"), "eps"), layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "logit_scale": self.logit_scale,
                "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": dict(l.mlp) if l.mlp is not None else None}
                           for l in self.layers]}


def _mixer_spec(cfg: NutopelConfig, l: LayerConfig) -> PartSpec:
    m, W, eps = l.mixer, cfg.width, cfg.norm_eps
    if l.type == "gla":
        return PartSpec("gated_linear_attention", {"hidden_size": W, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                                   "tau": m["tau"], "eps": eps, "decay_rank": m.get("decay_rank")})
    left, right = m["left"], m["right"]
    rot, mask = left.get("rot"), left.get("mask")
    attention = {"hidden_size": W, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"],
                 "scale": left["scale"], "eps": eps, "block": mask["size"] if mask else None, "max_positions": MAX_POSITIONS,
                 "rotary": {"theta": rot["base"], "rotary_dim": rot["dims"], "scaling": rot.get("scaling")} if rot else None}
    delta = {"hidden_size": W, "heads": right["heads"], "kv_heads": right["kv_heads"], "dim": right["dim"], "vdim": right["vdim"],
             "conv": right["conv"], "eps": eps}
    return PartSpec("side_by_side", {"hidden_size": W, "eps": eps, "left": {"kind": "normed_attention", "params": attention},
                                     "right": {"kind": "gated_delta", "params": delta}})


def _ffn_spec(cfg: NutopelConfig, mlp: dict) -> PartSpec:
    r = mlp["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "experts": r["experts"], "top": r["top"], "groups": g["count"],
                                       "keep": g["keep"], "scale": r["scale"], "expert_ff": mlp["expert"]["ff"],
                                       "shared_ff": (mlp.get("shared") or {}).get("ff", 0)})


def plan(cfg: NutopelConfig) -> ModelPlan:
    norm = PartSpec("group_rmsnorm", {"size": cfg.width, "groups": 1, "eps": cfg.norm_eps, "offset": 1.0})
    layers = []
    for i, l in enumerate(cfg.layers):
        parts = {"mixer_norm": PartEntry("norm", norm, "norm1"), "mixer": PartEntry("mixer", _mixer_spec(cfg, l), "mix")}
        if l.mlp is not None:
            parts["ffn_norm"] = PartEntry("norm", norm, "norm2")
            parts["ffn"] = PartEntry("feed_forward", _ffn_spec(cfg, l.mlp), "mlp")
        layers.append(LayerSpec(prefix=f"l{i}", parts=parts, block="pre_norm"))
    # the head's factor on the logits rides on the last norm's gain: head (s x) = s (head x)
    final = PartSpec("group_rmsnorm", {"size": cfg.width, "groups": 1, "eps": cfg.norm_eps, "offset": 1.0,
                                       "gain_scale": cfg.logit_scale})
    p = ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), run_list=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=final, final_norm_name="final.norm", head_name="head", position=None)
    p.validate()
    return p


def config_from_recipe(t: dict) -> dict:
    """A recipe's inline geometry carries config.json's own keys (``vocab``, ``width``, ``logit_scale``, ``norm``,
    ``layers``); a missing one raises KeyError naming it."""
    cfg = {k: t[k] for k in ("vocab", "width", "norm", "layers")}
    cfg["logit_scale"] = t.get("logit_scale", 1.0)
    cfg["architecture"] = NAME
    return cfg


register_architecture(Architecture(name=NAME, config_cls=NutopelConfig, plan=plan, aliases=("nutopel",),
                                   config_from_recipe=config_from_recipe), replace=True)
