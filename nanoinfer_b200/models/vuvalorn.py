"""The Vuvalorn architecture: config.json keys and tensor names.

A decoder whose layers are listed one by one in ``layers``.  Every layer is a sandwich: each sublayer
reads the stream through a norm and its output passes a second norm before it joins the stream.  The
mixer (``type`` "attention") is grouped-query attention whose queries and keys pass a short causal
convolution, a per-head RMS norm and a partial rotation of adjacent pairs, whose values are the
convolved keys, whose scores are capped by a tanh and whose heads are gated; the feed-forward
(``mlp``) is a capped gated unit ("dense"), a routed set of small gated units with identity experts
("moe"), or absent (null).  ``loop`` names a span of layers that runs several times in a row with
the same weights, every pass with a cache of its own and preceded by a learned vector added to the
stream.  The embedding is scaled, the output reuses the embedding's table and scales the logits.

Every size and every constant that may differ between models of the design is read here from
config.json; nothing is taken from a particular model.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, LayerSpec,
                                   MixerSpec, ModelConfig, NormSpec, PositionSpec, require)
from ..config.registry import register_architecture

NAME = "Vuvalorn"

# Positions are computed, not looked up, so nothing ends a sequence but the cache.
NO_POSITION_LIMIT = 1 << 30

# Constants the design fixes (they are parameters of the parts, so another design may choose others).
GATE_SLOPE = 1.702       # the dense unit's gate is g * sigmoid(GATE_SLOPE * g)
UP_SHIFT = 1.0           # ... and multiplies (up + UP_SHIFT)


def _mixer(i: int, layer: Dict[str, Any], eps: float) -> MixerSpec:
    kind = require(layer, "type", str)
    if kind != "attention":
        raise ConfigError(f"config.json: layers[{i}].type '{kind}' is not a mixer of this architecture (attention)")
    m = require(layer, "mixer", dict)
    heads, kv_heads, dim = require(m, "heads", int), require(m, "kv_heads", int), require(m, "dim", int)
    if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
        raise ConfigError(f"config.json: layers[{i}]: heads {heads} must be a positive multiple of kv_heads {kv_heads}")
    vdim = m.get("vdim", dim)
    if vdim != dim:
        raise ConfigError(f"config.json: layers[{i}]: the values are the keys, so vdim {vdim} must equal dim {dim}")
    rot = m.get("rot")
    if rot is None:
        position = PositionSpec(kind="none")
    else:
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: layers[{i}].mixer.rot must be an object or null")
        dims = require(rot, "dims", int)
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims {dims} must be even and at most dim {dim}")
        position = PositionSpec(kind="rope_exact", theta=require(rot, "base", float), rotary_dim=dims,
                                pairing="interleaved") if dims > 0 else PositionSpec(kind="none")
    taps = m.get("conv", 1)
    if not isinstance(taps, int) or isinstance(taps, bool) or taps < 1:
        raise ConfigError(f"config.json: layers[{i}].mixer.conv must be a positive number of taps")
    cap = m.get("softcap")
    extra = (("conv_taps", taps), ("norm_eps", eps), ("score_cap", float(cap) if cap else 0.0))
    return MixerSpec(kind="conv_key_attention", num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                     softmax_scale=require(m, "scale", float), position=position, extra=extra)


def _feed_forward(i: int, layer: Dict[str, Any]) -> Optional[FeedForwardSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
    kind = require(mlp, "kind", str)
    if kind == "dense":
        return FeedForwardSpec(kind="capped_glu", intermediate_size=require(mlp, "ff", int),
                               extra=(("limit", require(mlp, "limit", float)), ("gate_slope", GATE_SLOPE),
                                      ("up_shift", UP_SHIFT)))
    if kind == "moe":
        router = require(mlp, "router", dict)
        experts, top = require(router, "experts", int), require(router, "top", int)
        identity = router.get("identity") or 0
        if not isinstance(identity, int) or isinstance(identity, bool) or identity < 0:
            raise ConfigError(f"config.json: layers[{i}].mlp.router.identity must be a count")
        if experts < 0 or experts + identity <= 0 or not 0 < top <= experts + identity:
            raise ConfigError(f"config.json: layers[{i}].mlp.router: top {top} must lie in 1 .. experts + identity "
                              f"({experts} + {identity})")
        return FeedForwardSpec(kind="routed_experts", intermediate_size=require(require(mlp, "expert", dict), "ff", int),
                               extra=(("experts", experts), ("identity_experts", identity), ("top", top),
                                      ("choice_bias", True), ("renormalize", False)))
    raise ConfigError(f"config.json: layers[{i}].mlp.kind '{kind}' is not supported (dense, moe)")


def _schedule(n_layers: int, loop) -> Tuple[List[LayerRun], int]:
    """The order of runs: layers before the span once, the span ``times`` times (the first run of each
    pass takes stream input t), the rest once."""
    if loop is None:
        return [LayerRun(layer=i) for i in range(n_layers)], 0
    if not isinstance(loop, dict):
        raise ConfigError("config.json: 'loop' must be an object or null")
    start, stop, times = require(loop, "start", int), require(loop, "stop", int), require(loop, "times", int)
    if not 0 <= start <= stop <= n_layers or times < 1:
        raise ConfigError(f"config.json: loop {start}..{stop} x {times} does not fit {n_layers} layers")
    runs = [LayerRun(layer=i) for i in range(start)]
    for t in range(times):
        runs += [LayerRun(layer=i, stream_input=t if i == start else None) for i in range(start, stop)]
    runs += [LayerRun(layer=i) for i in range(stop, n_layers)]
    return runs, times


def parse_config(raw: Dict[str, Any]) -> ModelConfig:
    width, vocab = require(raw, "width", int), require(raw, "vocab", int)
    eps = require(require(raw, "norm", dict), "eps", float)
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw or not all(isinstance(x, dict) for x in layers_raw):
        raise ConfigError("config.json: 'layers' must be a non-empty list of objects")
    emb = raw.get("embedding") or {}
    if not isinstance(emb, dict):
        raise ConfigError("config.json: 'embedding' must be an object")
    emb_scale = float(emb["scale"]) if emb.get("scale") is not None else 1.0
    logit_scale = float(raw["logit_scale"]) if raw.get("logit_scale") is not None else 1.0
    norm = NormSpec(kind="rmsnorm", eps=eps)
    layers = []
    for i, layer in enumerate(layers_raw):
        ffn = _feed_forward(i, layer)
        layers.append(LayerSpec(mixer=_mixer(i, layer, eps), feed_forward=ffn, mixer_norm=norm,
                                ffn_norm=norm if ffn is not None else None, arrangement="sandwich_norm",
                                mixer_post_norm=norm, ffn_post_norm=norm if ffn is not None else None))
    schedule, passes = _schedule(len(layers), raw.get("loop"))
    return ModelConfig(
        architecture=NAME, hidden_size=width, vocab_size=vocab, max_position_embeddings=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tie_word_embeddings=True,
        embedding=EmbeddingSpec(kind="table", extra=(("row_scale", emb_scale),)),
        head=HeadSpec(kind="linear", tied=True, extra=(("logit_scale", logit_scale),)),
        stream_inputs=passes, raw=tuple(sorted((k, repr(v)) for k, v in raw.items())))


_LAYER_NORMS = {"mixer_norm": "norm1", "ffn_norm": "norm2", "mixer_post_norm": "norm1b", "ffn_post_norm": "norm2b"}


def tensor_name(scope: Tuple, slot: str) -> str:
    if scope == ("embedding",):
        return "embed"
    if scope == ("final_norm",):
        return "final.norm"
    if scope == ("stream_inputs",):
        return "loop.step"
    if scope[0] == "layer":
        _, i, what = scope
        if what == "mixer":
            return f"l{i}.mix.{slot}"
        if what == "feed_forward":
            return f"l{i}.mlp.{slot}"
        if what in _LAYER_NORMS:
            return f"l{i}.{_LAYER_NORMS[what]}"
    raise ConfigError(f"{NAME}: no tensor name for scope {scope} slot '{slot}'")


register_architecture(NAME, parse_config, tensor_name, replace=True)
