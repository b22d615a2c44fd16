"""The Tazulix architecture: config.json keys and tensor names.

A decoder whose layers are listed one by one in ``layers``; every layer is pre-norm
(x += mixer(norm1(x)); x += ff(norm2(x)), the second half absent when ``mlp`` is null).  The mixer
(``type``) is either

  "attention"   grouped-query attention with biased projections, an RMS norm over the WHOLE query
                projection and over the whole key projection (before the heads are split), a partial
                rotation of the pairs (i, i + dims / 2) with ramp-scaled frequencies, a score scale from
                the configuration, causal softmax; keys and values may differ in size;
  "lightning"   linear attention with a fixed decay per head and a matrix state per request, silu on
                queries, keys and values, an RMS norm over all heads and a sigmoid gate.

The feed-forward (``mlp.kind``) is "dense" (W_down relu(W_up h)^2) or "moe" (sigmoid router, the chosen
experts read the token's input multiplied by their score, capped gated units, an optional shared unit).
``loop`` names a span of layers that runs several times in a row with the same weights; every pass has
caches and states of its own and begins with x <- W_in [x; x0], x0 being the embedding's output.  The
embedding is scaled; the output has a matrix of its own.

Every size and every constant that may differ between models of the design is read here from
config.json; nothing is taken from a particular model.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, LayerSpec,
                                   MixerSpec, ModelConfig, NormSpec, PositionSpec, RopeScaling, require)
from ..config.registry import register_architecture

NAME = "Tazulix"

# Positions are computed, not looked up, so nothing ends a sequence but the cache.
NO_POSITION_LIMIT = 1 << 30

# Constants the design fixes (they are parameters of the parts, so another design may choose others).
GATE_SLOPE = 1.702       # an expert's gate is g * sigmoid(GATE_SLOPE * g)
UP_SHIFT = 1.0           # ... and multiplies (up + UP_SHIFT)


def _count(raw: Dict[str, Any], key: str, where: str) -> int:
    n = require(raw, key, int)
    if n <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be positive (found {n})")
    return n


def _position(i: int, rot, dim: int) -> PositionSpec:
    if rot is None:
        return PositionSpec(kind="none")
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: layers[{i}].mixer.rot must be an object or null")
    dims = require(rot, "dims", int)
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims {dims} must be even and at most dim {dim}")
    if dims == 0:
        return PositionSpec(kind="none")
    scaling = None
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: layers[{i}].mixer.rot.scaling must be an object or null")
        scaling = RopeScaling(rope_type="yarn", factor=require(sc, "factor", float),
                              low_freq_factor=require(sc, "slow", float), high_freq_factor=require(sc, "fast", float),
                              original_max_position_embeddings=require(sc, "original", float))
    return PositionSpec(kind="rope_yarn", theta=require(rot, "base", float), rotary_dim=dims, pairing="half",
                        scaling=scaling)


def _mixer(i: int, layer: Dict[str, Any], eps: float) -> MixerSpec:
    kind = require(layer, "type", str)
    m = require(layer, "mixer", dict)
    where = f"layers[{i}].mixer"
    heads, dim = _count(m, "heads", where), _count(m, "dim", where)
    vdim = _count(m, "vdim", where) if m.get("vdim") is not None else dim
    if kind == "attention":
        kv_heads = _count(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: heads {heads} must be a multiple of kv_heads {kv_heads}")
        return MixerSpec(kind="normed_qk_attention", num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                         softmax_scale=require(m, "scale", float), position=_position(i, m.get("rot"), dim),
                         extra=(("value_dim", vdim), ("norm_eps", eps), ("bias", True), ("qk_norm", True)))
    if kind == "lightning":
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or \
                not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
            raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
        return MixerSpec(kind="lightning", num_heads=heads, num_kv_heads=heads, head_dim=dim,
                         position=PositionSpec(kind="none"),
                         extra=(("value_dim", vdim), ("decay", tuple(float(x) for x in decay)), ("norm_eps", eps)))
    raise ConfigError(f"config.json: layers[{i}].type '{kind}' is not a mixer of this architecture "
                      f"(attention, lightning)")


def _feed_forward(i: int, layer: Dict[str, Any]) -> Optional[FeedForwardSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
    kind = require(mlp, "kind", str)
    where = f"layers[{i}].mlp"
    if kind == "dense":
        return FeedForwardSpec(kind="relu2", intermediate_size=_count(mlp, "ff", where))
    if kind == "moe":
        router, expert = require(mlp, "router", dict), require(mlp, "expert", dict)
        experts, top = _count(router, "experts", where + ".router"), _count(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: top {top} exceeds the {experts} experts")
        extra = [("experts", experts), ("top", top), ("scores", "sigmoid"), ("weight_on_input", True),
                 ("limit", require(expert, "limit", float)), ("gate_slope", GATE_SLOPE), ("up_shift", UP_SHIFT)]
        shared = mlp.get("shared")
        if shared is not None:
            if not isinstance(shared, dict):
                raise ConfigError(f"config.json: {where}.shared must be an object or null")
            extra += [("shared_ff", _count(shared, "ff", where + ".shared")),
                      ("shared_limit", require(shared, "limit", float))]
        return FeedForwardSpec(kind="routed_experts", intermediate_size=_count(expert, "ff", where + ".expert"),
                               extra=tuple(extra))
    raise ConfigError(f"config.json: {where}.kind '{kind}' is not supported (dense, moe)")


def _schedule(n_layers: int, loop) -> Tuple[List[LayerRun], int]:
    """The order of runs: layers before the span once, the span ``times`` times (the first run of each
    pass is marked: the stream is projected together with the embedding's output right before it), the
    rest once."""
    if loop is None:
        return [LayerRun(layer=i) for i in range(n_layers)], 0
    if not isinstance(loop, dict):
        raise ConfigError("config.json: 'loop' must be an object or null")
    start, stop, times = require(loop, "start", int), require(loop, "stop", int), require(loop, "times", int)
    if not 0 <= start < stop <= n_layers or times < 1:
        raise ConfigError(f"config.json: loop {start}..{stop} x {times} does not fit {n_layers} layers")
    runs = [LayerRun(layer=i) for i in range(start)]
    for t in range(times):
        runs += [LayerRun(layer=i, stream_input=t if i == start else None) for i in range(start, stop)]
    runs += [LayerRun(layer=i) for i in range(stop, n_layers)]
    return runs, times


def parse_config(raw: Dict[str, Any]) -> ModelConfig:
    width, vocab = _count(raw, "width", "config"), _count(raw, "vocab", "config")
    eps = require(require(raw, "norm", dict), "eps", float)
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw or not all(isinstance(x, dict) for x in layers_raw):
        raise ConfigError("config.json: 'layers' must be a non-empty list of objects")
    emb = raw.get("embedding") or {}
    if not isinstance(emb, dict):
        raise ConfigError("config.json: 'embedding' must be an object")
    emb_scale = float(emb["scale"]) if emb.get("scale") is not None else 1.0
    norm = NormSpec(kind="rmsnorm", eps=eps)
    layers = []
    for i, layer in enumerate(layers_raw):
        ffn = _feed_forward(i, layer)
        layers.append(LayerSpec(mixer=_mixer(i, layer, eps), feed_forward=ffn, mixer_norm=norm,
                                ffn_norm=norm if ffn is not None else None, arrangement="pre_norm"))
    schedule, passes = _schedule(len(layers), raw.get("loop"))
    return ModelConfig(
        architecture=NAME, hidden_size=width, vocab_size=vocab, max_position_embeddings=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tie_word_embeddings=False,
        embedding=EmbeddingSpec(kind="table", extra=(("row_scale", emb_scale),)),
        head=HeadSpec(kind="linear", tied=False),
        stream_inputs=passes, stream_input_kind="project_with_embedding" if passes else "row",
        raw=tuple(sorted((k, repr(v)) for k, v in raw.items())))


_LAYER_NORMS = {"mixer_norm": "norm1", "ffn_norm": "norm2"}


def tensor_name(scope: Tuple, slot: str) -> str:
    if scope == ("embedding",):
        return "embed"
    if scope == ("lm_head",):
        return "head"
    if scope == ("final_norm",):
        return "final.norm"
    if scope == ("stream_inputs",):
        return "loop.in"
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
