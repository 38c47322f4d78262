"""The Runevik architecture: config.json keys and tensor names.

A decoder whose layers are listed one by one in ``layers``: each names its mixer (``type``: "delta", the
gated delta rule, or "latent_attention", attention over one compressed vector per token, which a later
layer may borrow through ``kv_from``) with the mixer's sizes, and its feed-forward (``mlp``: dense with the
PolyNorm activation, or null).  A layer is parallel - one RMS norm with a single gain, read by mixer and
feed-forward alike - and is followed by a per-layer token input when ``token_side`` gives its width.  The
embedding adds a sinusoidal position vector; the output is the same norm and a linear head.

Every size and every constant that may differ between models of the design is read here from
config.json; nothing is taken from a particular model.
"""
from __future__ import annotations

from typing import Any, Dict, Tuple

from ..config.model_config import (ConfigError, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, LayerSpec,
                                   MixerSpec, ModelConfig, NormSpec, PositionSpec, optional, require)
from ..config.registry import register_architecture

NAME = "Runevik"

# Positions are computed, not looked up, so nothing ends a sequence but the cache.
NO_POSITION_LIMIT = 1 << 30


def _mixer(i: int, layer: Dict[str, Any], eps: float, layers) -> Tuple[MixerSpec, Any]:
    kind = require(layer, "type", str)
    m = require(layer, "mixer", dict)
    none = PositionSpec(kind="none")
    if kind == "delta":
        heads, kv_heads = require(m, "heads", int), require(m, "kv_heads", int)
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(f"config.json: layers[{i}]: heads {heads} must be a positive multiple of kv_heads {kv_heads}")
        extra = (("value_dim", require(m, "vdim", int)), ("conv_taps", require(m, "conv", int)), ("norm_eps", eps))
        return MixerSpec(kind="gated_delta", num_heads=heads, num_kv_heads=kv_heads, head_dim=require(m, "dim", int),
                         position=none, extra=extra), None
    if kind == "latent_attention":
        rank = require(m, "kv_rank", int)
        source = m.get("kv_from")
        if source is not None:
            if not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from must name an earlier layer")
            other = layers[source]
            if other.get("type") != "latent_attention" or other.get("mixer", {}).get("kv_from") is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={source} must name a latent_attention "
                                  f"layer with a latent of its own")
            if other["mixer"].get("kv_rank") != rank:
                raise ConfigError(f"config.json: layers[{i}] and layers[{source}] share a latent but differ in kv_rank")
        extra = (("value_dim", require(m, "vdim", int)), ("latent_rank", rank), ("own_latent", source is None),
                 ("norm_eps", eps))
        return MixerSpec(kind="latent_attention", num_heads=require(m, "heads", int), num_kv_heads=1,
                         head_dim=require(m, "dim", int), softmax_scale=require(m, "scale", float), position=none,
                         extra=extra), source
    raise ConfigError(f"config.json: layers[{i}].type '{kind}' is not a mixer of this architecture "
                      f"(delta, latent_attention)")


def _feed_forward(i: int, layer: Dict[str, Any], eps: float):
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
    kind = require(mlp, "kind", str)
    if kind != "dense":
        raise ConfigError(f"config.json: layers[{i}].mlp.kind '{kind}' is not supported (dense)")
    return FeedForwardSpec(kind="polynorm", intermediate_size=require(mlp, "ff", int), extra=(("eps", eps),))


def parse_config(raw: Dict[str, Any]) -> ModelConfig:
    width, vocab = require(raw, "width", int), require(raw, "vocab", int)
    eps = require(require(raw, "norm", dict), "eps", float)
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw or not all(isinstance(x, dict) for x in layers_raw):
        raise ConfigError("config.json: 'layers' must be a non-empty list of objects")
    side = raw.get("token_side")
    if side is not None and not isinstance(side, dict):
        raise ConfigError("config.json: 'token_side' must be an object or null")
    side_dim = require(side, "dim", int) if side is not None else 0
    if side_dim < 0:
        raise ConfigError("config.json: token_side.dim must not be negative")
    norm = NormSpec(kind="rmsnorm_scalar", eps=eps)
    layers, schedule = [], []
    for i, layer in enumerate(layers_raw):
        mixer, source = _mixer(i, layer, eps, layers_raw)
        extra = (("token_input_dim", side_dim), ("token_input_index", i), ("token_input_eps", eps)) if side_dim else ()
        layers.append(LayerSpec(mixer=mixer, feed_forward=_feed_forward(i, layer, eps), mixer_norm=norm, ffn_norm=None,
                                arrangement="parallel", extra=extra))
        schedule.append(LayerRun(layer=i, cache_of=source))
    emb_extra = (("layer_inputs", side_dim * len(layers)),) if side_dim else ()
    return ModelConfig(
        architecture=NAME, hidden_size=width, vocab_size=vocab, max_position_embeddings=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tie_word_embeddings=False,
        embedding=EmbeddingSpec(kind="table_sinusoid", extra=emb_extra), head=HeadSpec(kind="linear"),
        raw=tuple(sorted((k, repr(v)) for k, v in raw.items())))


def tensor_name(scope: Tuple, slot: str) -> str:
    if scope == ("embedding",):
        return {"weight": "embed", "layer_inputs": "side.embed"}[slot]
    if scope == ("lm_head",):
        return "head"
    if scope == ("final_norm",):
        return "final.norm"
    if scope[0] == "layer":
        _, i, what = scope
        if what == "mixer":
            return f"l{i}.mix.{slot}"
        if what == "feed_forward":
            return f"l{i}.mlp.{slot}"
        if what == "mixer_norm":
            return f"l{i}.norm1"
        if what == "block":
            return f"l{i}.side.{slot}"
    raise ConfigError(f"{NAME}: no tensor name for scope {scope} slot '{slot}'")


register_architecture(NAME, parse_config, tensor_name, replace=True)
