"""Architecture builder for ``Dulisun``: a decoder whose layers are listed one by one in
``config.json``.

The configuration names its architecture as a string (``"architecture": "Dulisun"``) and gives
``vocab``, ``width``, ``norm.eps`` and ``layers``: per layer its ``type`` (the kind of mixer),
the mixer's sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (null: the
layer has none).  The model:

* embedding table, then the model's norm on the row; the head multiplies by the same table;
* every norm is an RMS norm whose stored weight lies around zero (it multiplies by 1 + w);
* a layer sums norm(sublayer(x)) into the stream, for the mixer and then for the feed-forward:
  the norm stands on the sublayer's output, the sublayer reads the stream itself;
* mixer ``attention``: grouped-query attention without a value projection (a value is its key as
  projected), rotation of neighbouring pairs over the first ``rot.dims`` dimensions with base
  ``rot.base``, q and k brought to unit root mean square after the rotation, scores times
  ``scale``, a chunk mask of ``mask.size`` positions, a learned softmax sink per head;
* feed-forward ``moe``: ``router.experts`` experts of hidden size ``expert.ff`` with the erf gelu,
  ``router.top`` per token chosen by softmax score among the best ``router.groups.keep`` of
  ``router.groups.count`` groups, weighted by their scores as they are, plus a shared expert of
  hidden size ``shared.ff``.

This file is the only place that knows the configuration's keys and the checkpoint's tensor
names (``embed``, ``embed.norm``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|sink|o``,
``l<i>.mlp.router``, ``l<i>.mlp.e<j>.up|down``, ``l<i>.mlp.shared.up|down``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_run_list
from ..registry import register_architecture

# The design sets no limit on positions; the engine's tables need one.  EngineConfig.max_context overrides it.
DEFAULT_MAX_POSITION = 131072


@dataclass(frozen=True)
class DulisunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITION
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def _need(obj: Any, key: str, where: str, kind=None):
    if not isinstance(obj, Mapping) or key not in obj or obj[key] is None:
        raise ConfigError(f"config.json: {where}.{key} is missing")
    v = obj[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    elif kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        v = float(v)
    return v


def _attention_parts(i: int, mixer: Mapping[str, Any], width: int, eps: float):
    where = f"layers[{i}].mixer"
    dim = _need(mixer, "dim", where, int)
    rot = mixer.get("rot")
    if rot and rot.get("dims"):
        position = PartSpec("rotary", {"head_dim": dim, "theta": _need(rot, "base", where + ".rot", float),
                                       "rotary_dim": _need(rot, "dims", where + ".rot", int), "pairing": "interleaved",
                                       "theta_as_float32": False})
    else:
        position = PartSpec("none", {})
    mask = mixer.get("mask") or {}
    params = {
        "hidden_size": width, "num_heads": _need(mixer, "heads", where, int),
        "num_kv_heads": int(mixer.get("kv_heads") or mixer["heads"]), "head_dim": dim,
        "value_dim": int(mixer.get("vdim") or dim), "scale": _need(mixer, "scale", where, float),
        "chunk": int(mask.get("size") or 0), "sink": True, "unit_qk": True, "unit_eps": eps, "values_from_keys": True,
    }
    return position, PartSpec("chunked_sink_attention", params)


def _moe_part(i: int, mlp: Mapping[str, Any], width: int) -> PartSpec:
    where = f"layers[{i}].mlp"
    kind = mlp.get("kind", "moe")
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r}: this design has the feed-forward 'moe'")
    router = _need(mlp, "router", where)
    expert = _need(mlp, "expert", where)
    groups = router.get("groups") or {}
    shared = mlp.get("shared") or {}
    return PartSpec("routed_experts", {
        "hidden_size": width, "expert_ff": _need(expert, "ff", where + ".expert", int),
        "num_experts": _need(router, "experts", where + ".router", int), "top": _need(router, "top", where + ".router", int),
        "group_count": int(groups.get("count") or 1), "group_keep": int(groups.get("keep") or groups.get("count") or 1),
        "shared_ff": int(shared.get("ff") or 0), "act": expert.get("act", "gelu"), "shared_act": shared.get("act"),
        "renormalise": False,
    })


_MIXERS = {"attention": _attention_parts}


def spec_from_config(cfg: DulisunConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "weight_offset": 1.0})
    layers = []
    for i, layer in enumerate(cfg.layers):
        kind = layer.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: layers[{i}].type {kind!r}: this design has the mixers {sorted(_MIXERS)}")
        position, mixer = _MIXERS[kind](i, _need(layer, "mixer", f"layers[{i}]"), cfg.hidden_size, cfg.norm_eps)
        names = {"norm_mixer.weight": "norm1", "mixer.q_proj": "mix.q", "mixer.k_proj": "mix.k", "mixer.o_proj": "mix.o",
                 "mixer.sink": "mix.sink"}
        mlp = layer.get("mlp")
        ff = None
        if mlp:
            ff = _moe_part(i, mlp, cfg.hidden_size)
            names.update({"norm_ff.weight": "norm2", "feed_forward.router": "mlp.router",
                          "feed_forward.shared.up": "mlp.shared.up", "feed_forward.shared.down": "mlp.shared.down"})
            for e in range(ff.params["num_experts"]):
                names[f"feed_forward.experts.{e}.up"] = f"mlp.e{e}.up"
                names[f"feed_forward.experts.{e}.down"] = f"mlp.e{e}.down"
        layers.append(LayerSpec(block="branchnorm" if ff is not None else "branchnorm_mixer", mixer=mixer, feed_forward=ff,
                                norm=norm, position=position, prefix=f"l{i}.", names=names))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        layers=tuple(layers), run_list=default_run_list(len(layers)),
        embedding=PartSpec("table_normed", {"name": "embed", "names": {"norm.weight": "embed.norm"},
                                            "norm": {"kind": "rmsnorm", "eps": cfg.norm_eps, "weight_offset": 1.0}}),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.norm_eps, "weight_offset": 1.0, "name": "final.norm"}),
        head=PartSpec("linear", {"tied": True}),
        max_position=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.eos_token_ids),
    )


def config_from_dict(raw: Mapping[str, Any], generation_config: Optional[Mapping[str, Any]] = None) -> DulisunConfig:
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: layers must be a non-empty list")
    eos = ()
    for src in (generation_config, raw):
        v = src.get("eos_token_id") if isinstance(src, Mapping) else None
        if v is not None:
            eos = tuple(int(t) for t in (v if isinstance(v, (list, tuple)) else [v]))
            break
    return DulisunConfig(
        architecture="Dulisun", vocab_size=_need(raw, "vocab", "config", int), hidden_size=_need(raw, "width", "config", int),
        norm_eps=_need(_need(raw, "norm", "config"), "eps", "config.norm", float), layers=tuple(layers),
        max_position_embeddings=DEFAULT_MAX_POSITION, eos_token_ids=eos,
    )


@register_architecture("Dulisun")
def _build(raw, generation_config=None, strict=False):
    cfg = config_from_dict(raw, generation_config)
    return cfg, spec_from_config(cfg)
