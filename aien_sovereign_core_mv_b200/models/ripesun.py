"""Architecture builder for ``Ripesun``: a decoder that mixes, layer by layer, attention over a cached latent,
linear attention with decay, and a gated recurrence, all listed one by one in ``config.json``.

The configuration names its architecture as a string (``"architecture": "Ripesun"``) and gives ``vocab``, ``width``,
``norm.eps``, ``embedding.scale``, ``residual_mult``, ``logit_softcap``, ``token_side.dim`` and ``layers``: per layer its
``type`` (the kind of mixer), the mixer's sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (null:
the layer has none).  In this file's notation, with the float32 stream x, m = ``residual_mult`` and every norm N an RMS
norm with a plain weight, x / sqrt(mean x^2 + eps) * w:

* x = embed[token] * ``embedding.scale``; logits = c tanh(head N_final(x) / c) with c = ``logit_softcap``;
* a layer: x <- x + m N_1b(mixer(N_1(x))); x <- x + m N_2b(ff(N_2(x))); then the token's side input:
  e = the layer's ``token_side.dim`` columns of side.embed[token], y = W_proj (gelu_tanh(W_gate x) * e),
  x <- x + m N_side(y);
* mixer ``latent_attention``: see :class:`~..parts.latent_attention.LatentAttention`; ``kv_from``: j makes the layer read
  the cache rows of layer j (which has its own key/value projection) instead of writing its own;
* mixer ``lightning``: see :class:`~..parts.recurrent.DecayLinearAttention`; ``decay`` lists one value per head;
* mixer ``mingru``: see :class:`~..parts.recurrent.GatedRecurrence`;
* feed-forward ``dense``: W_down gelu_tanh(W_up h).

This file is the only place that knows the configuration's keys and the checkpoint's tensor names (``embed``,
``side.embed``, ``final.norm``, ``head``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``l<i>.side.gate|proj|norm``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture

# The design sets no limit on positions; the engine's tables need one.  EngineConfig.max_context overrides it.
DEFAULT_MAX_POSITION = 131072


@dataclass(frozen=True)
class RipesunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    logit_softcap: float
    side_dim: int
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


def _opt_number(obj: Any, key: str, default: float) -> float:
    v = obj.get(key) if isinstance(obj, Mapping) else None
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key} must be a number, got {v!r}")
    return float(v)


def _latent_attention(i: int, mixer: Mapping[str, Any], width: int, eps: float, cache_window: int):
    where = f"layers[{i}].mixer"
    rot_dim = int(mixer.get("rot_dim") or 0)
    rot = mixer.get("rot") or {}
    if rot_dim and rot.get("dims"):
        position = PartSpec("rotary", {"head_dim": rot_dim, "theta": _need(rot, "base", where + ".rot", float),
                                       "rotary_dim": _need(rot, "dims", where + ".rot", int), "pairing": "interleaved",
                                       "theta_as_float32": False})
    else:
        position = PartSpec("none", {})
    mask = mixer.get("mask") or {}
    params = {
        "hidden_size": width, "num_heads": _need(mixer, "heads", where, int), "head_dim": _need(mixer, "dim", where, int),
        "rot_dim": rot_dim, "value_dim": int(mixer.get("vdim") or mixer["dim"]), "kv_rank": _need(mixer, "kv_rank", where, int),
        "q_rank": _need(mixer, "q_rank", where, int), "scale": _need(mixer, "scale", where, float),
        "window": int(mask.get("size") or 0), "cache_window": int(cache_window), "sink": True, "norm_eps": eps,
        "own_cache": mixer.get("kv_from") is None,
    }
    names = {"mixer.dq_proj": "mix.dq", "mixer.dq_norm": "mix.dq.norm", "mixer.uq_proj": "mix.uq", "mixer.dkv_proj": "mix.dkv",
             "mixer.dkv_norm": "mix.dkv.norm", "mixer.uk_proj": "mix.uk", "mixer.uv_proj": "mix.uv", "mixer.sink": "mix.sink",
             "mixer.o_proj": "mix.o"}
    return position, PartSpec("latent_attention", params), names


def _lightning(i: int, mixer: Mapping[str, Any], width: int, eps: float, _cw: int):
    where = f"layers[{i}].mixer"
    heads = _need(mixer, "heads", where, int)
    decay = _need(mixer, "decay", where)
    if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
        raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
    params = {"hidden_size": width, "num_heads": heads, "head_dim": _need(mixer, "dim", where, int),
              "value_dim": int(mixer.get("vdim") or mixer["dim"]), "decay": tuple(float(d) for d in decay), "norm_eps": eps}
    names = {"mixer.q_proj": "mix.q", "mixer.k_proj": "mix.k", "mixer.v_proj": "mix.v", "mixer.g_proj": "mix.g",
             "mixer.o_proj": "mix.o", "mixer.norm": "mix.norm"}
    return PartSpec("none", {}), PartSpec("decay_linear_attention", params), names


def _mingru(i: int, mixer: Mapping[str, Any], width: int, eps: float, _cw: int):
    params = {"hidden_size": width, "width": _need(mixer, "width", f"layers[{i}].mixer", int), "bias": True}
    names = {"mixer.z_proj": "mix.z", "mixer.z_bias": "mix.z.b", "mixer.x_proj": "mix.x", "mixer.x_bias": "mix.x.b",
             "mixer.g_proj": "mix.g", "mixer.o_proj": "mix.o"}
    return PartSpec("none", {}), PartSpec("gated_recurrence", params), names


_MIXERS = {"latent_attention": _latent_attention, "lightning": _lightning, "mingru": _mingru}


def _dense_part(i: int, mlp: Mapping[str, Any], width: int) -> PartSpec:
    where = f"layers[{i}].mlp"
    kind = mlp.get("kind", "dense")
    if kind != "dense":
        raise ConfigError(f"config.json: {where}.kind {kind!r}: this design has the feed-forward 'dense'")
    return PartSpec("mlp_act", {"hidden_size": width, "intermediate_size": _need(mlp, "ff", where, int), "act": "gelu_tanh"})


def _cache_sources(layers) -> Dict[int, int]:
    """layer -> the layer whose cache rows it reads (itself when it writes its own); checked."""
    src: Dict[int, int] = {}
    for i, layer in enumerate(layers):
        if layer.get("type") != "latent_attention":
            continue
        mixer = _need(layer, "mixer", f"layers[{i}]")
        j = mixer.get("kv_from")
        if j is None:
            src[i] = i
            continue
        where = f"layers[{i}].mixer.kv_from"
        if isinstance(j, bool) or not isinstance(j, int) or not (0 <= j < i):
            raise ConfigError(f"config.json: {where} must name an earlier layer, got {j!r}")
        other = layers[j]
        if other.get("type") != "latent_attention" or (other.get("mixer") or {}).get("kv_from") is not None:
            raise ConfigError(f"config.json: {where} names layer {j}, which has no key/value projection of its own")
        om = other["mixer"]
        for key in ("kv_rank", "rot_dim"):
            if int(om.get(key) or 0) != int(mixer.get(key) or 0):
                raise ConfigError(f"config.json: {where}: layer {j} has another {key}")
        src[i] = j
    return src


def spec_from_config(cfg: RipesunConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps})
    src = _cache_sources(cfg.layers)
    # a shared cache keeps what the widest window among its readers needs; one reader without a window keeps all
    windows: Dict[int, list] = {}
    for i, j in src.items():
        mask = (cfg.layers[i]["mixer"].get("mask") or {})
        windows.setdefault(j, []).append(int(mask.get("size") or 0))
    keep = {j: (0 if min(ws) == 0 else max(ws)) for j, ws in windows.items()}
    layers, runs = [], []
    for i, layer in enumerate(cfg.layers):
        kind = layer.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: layers[{i}].type {kind!r}: this design has the mixers {sorted(_MIXERS)}")
        position, mixer, names = _MIXERS[kind](i, _need(layer, "mixer", f"layers[{i}]"), cfg.hidden_size, cfg.norm_eps,
                                               keep.get(src.get(i, i), 0))
        if kind == "latent_attention" and mixer.params["window"] == 0 and mixer.params["cache_window"] != 0:
            raise ConfigError(f"config.json: layers[{i}] sees every position but shares a cache that keeps a window")
        names = dict(names)
        names.update({"norm_in.weight": "norm1", "norm_out.weight": "norm1b"})
        mlp = layer.get("mlp")
        ff = None
        if mlp:
            ff = _dense_part(i, mlp, cfg.hidden_size)
            names.update({"norm_ff_in.weight": "norm2", "norm_ff_out.weight": "norm2b", "feed_forward.up": "mlp.up",
                          "feed_forward.down": "mlp.down"})
        block_params: Dict[str, Any] = {"residual_mult": cfg.residual_mult}
        if cfg.side_dim > 0:
            block_params["side"] = {"kind": "gated_token_table", "hidden_size": cfg.hidden_size, "dim": cfg.side_dim,
                                    "column": i * cfg.side_dim, "eps": cfg.norm_eps}
        layers.append(LayerSpec(block="sandwich" if ff is not None else "sandwich_mixer", mixer=mixer, feed_forward=ff, norm=norm,
                                position=position, prefix=f"l{i}.", names=names, block_params=block_params))
        runs.append(RunEntry(layer=i, cache=src.get(i, i), writes_cache=src.get(i, i) == i))
    embedding = {"name": "embed", "scale": cfg.embedding_scale}
    if cfg.side_dim > 0:
        embedding.update({"side_width": cfg.side_dim * len(cfg.layers), "names": {"side": "side.embed"}})
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        layers=tuple(layers), run_list=tuple(runs), embedding=PartSpec("table", embedding),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.norm_eps, "name": "final.norm"}),
        head=PartSpec("linear", {"tied": False, "name": "head", "softcap": cfg.logit_softcap}),
        max_position=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.eos_token_ids),
    )


def config_from_dict(raw: Mapping[str, Any], generation_config: Optional[Mapping[str, Any]] = None) -> RipesunConfig:
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: layers must be a non-empty list")
    eos = ()
    for source in (generation_config, raw):
        v = source.get("eos_token_id") if isinstance(source, Mapping) else None
        if v is not None:
            eos = tuple(int(t) for t in (v if isinstance(v, (list, tuple)) else [v]))
            break
    side = raw.get("token_side") or {}
    side_dim = side.get("dim") or 0
    if isinstance(side_dim, bool) or not isinstance(side_dim, int) or side_dim < 0:
        raise ConfigError(f"config.json: token_side.dim must be a positive integer, got {side_dim!r}")
    cap = _opt_number(raw, "logit_softcap", 0.0)
    if cap < 0:
        raise ConfigError(f"config.json: logit_softcap must not be negative, got {cap!r}")
    return RipesunConfig(
        architecture="Ripesun", vocab_size=_need(raw, "vocab", "config", int), hidden_size=_need(raw, "width", "config", int),
        norm_eps=_need(_need(raw, "norm", "config"), "eps", "config.norm", float),
        embedding_scale=_opt_number(raw.get("embedding") or {}, "scale", 1.0), residual_mult=_opt_number(raw, "residual_mult", 1.0),
        logit_softcap=cap, side_dim=int(side_dim), layers=tuple(layers),
        max_position_embeddings=DEFAULT_MAX_POSITION, eos_token_ids=eos,
    )


@register_architecture("Ripesun")
def _build(raw, generation_config=None, strict=False):
    cfg = config_from_dict(raw, generation_config)
    return cfg, spec_from_config(cfg)
