"""The Mobatar architecture: config.json keys and tensor names.

A decoder whose layers are listed one by one in ``layers``.  In every layer the sublayers read the stream itself and
only their outputs are normed: x += norm1(mixer(x)); x += norm2(ff(x)), the second half absent when ``mlp`` is null.
The norms are RMS norms whose weight is stored around zero (the gain is 1 + w).  The mixer (``type``) is one of

  "attention"         grouped-query attention: rotation of the pairs (i, i + dims / 2) with llama3-scaled frequencies,
                      then every head of q and k divided by its own root mean square; causal; a softmax with one added
                      to its denominator; keys and values may differ in size;
  "latent_attention"  attention over one compressed vector per token plus one rotated key part that all heads share
                      (adjacent pairs rotated); a token sees itself and the ``mask.size`` - 1 tokens before it;
  "parallel"          two mixers that read the same input, their outputs added with a scale each: on the left
                      grouped-query attention with an RMS norm over the WHOLE query and key projections, linearly
                      scaled rotary frequencies, a mask of chunks of ``mask.size`` positions and a sigmoid gate per
                      head; on the right retention - linear attention with a fixed decay per head, rotated queries and
                      keys, a per-head RMS norm of the read-out and a silu gate.

The feed-forward (``mlp.kind`` "dense") is a capped gated unit with biases on all three projections.  A layer with
``weights_of``: j runs with layer j's weights and a cache or state of its own.  The embedding adds a row of a second
table chosen by a hash of the token and the one before it (``embedding.bigram``).  The output has a matrix of its own.

Every size and every constant that may differ between models of the design is read here from config.json; nothing is
taken from a particular model.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, LayerSpec,
                                   MixerSpec, ModelConfig, NormSpec, PositionSpec, RopeScaling, require)
from ..config.registry import register_architecture

NAME = "Mobatar"

# Positions are computed, not looked up, so nothing ends a sequence but the cache.
NO_POSITION_LIMIT = 1 << 30

# Constants the design fixes (they are parameters of the parts, so another design may choose others).
GATE_SLOPE = 1.702       # the dense unit's gate is g * sigmoid(GATE_SLOPE * g)
UP_SHIFT = 1.0           # ... and multiplies (up + UP_SHIFT)


def _count(raw: Dict[str, Any], key: str, where: str) -> int:
    n = require(raw, key, int)
    if n <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be positive (found {n})")
    return n


def _position(where: str, rot, dim: int, pairing: str) -> PositionSpec:
    """``rot``: {base, dims, scaling}; scaling {factor} divides every frequency, scaling {factor, low, high, original}
    is the llama3 rule, no scaling leaves them."""
    if rot is None:
        return PositionSpec(kind="none")
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}.rot must be an object or null")
    dims = require(rot, "dims", int)
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most {dim}")
    if dims == 0:
        return PositionSpec(kind="none")
    scaling = None
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
        factor = require(sc, "factor", float)
        if any(sc.get(k) is not None for k in ("original", "low", "high")):
            scaling = RopeScaling(rope_type="llama3", factor=factor, low_freq_factor=require(sc, "low", float),
                                  high_freq_factor=require(sc, "high", float),
                                  original_max_position_embeddings=require(sc, "original", float))
        else:
            scaling = RopeScaling(rope_type="linear", factor=factor, low_freq_factor=1.0, high_freq_factor=1.0,
                                  original_max_position_embeddings=0)
    return PositionSpec(kind="rope_scaled", theta=require(rot, "base", float), rotary_dim=dims, pairing=pairing,
                        scaling=scaling)


def _mask_size(where: str, m: Dict[str, Any]) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}.mask must be an object or null")
    return _count(mask, "size", where + ".mask")


def _heads(where: str, m: Dict[str, Any]) -> Tuple[int, int, int, int]:
    heads, dim = _count(m, "heads", where), _count(m, "dim", where)
    kv_heads = _count(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
    vdim = _count(m, "vdim", where) if m.get("vdim") is not None else dim
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: heads {heads} must be a multiple of kv_heads {kv_heads}")
    return heads, kv_heads, dim, vdim


def _sink_attention(where: str, m: Dict[str, Any], eps: float) -> MixerSpec:
    heads, kv_heads, dim, vdim = _heads(where, m)
    return MixerSpec(kind="normed_qk_attention", num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                     softmax_scale=require(m, "scale", float), position=_position(where, m.get("rot"), dim, "half"),
                     extra=(("value_dim", vdim), ("norm_eps", eps), ("bias", False), ("qk_norm", False),
                            ("head_unit_norm", True), ("sink", True)))


def _chunked_attention(where: str, m: Dict[str, Any], eps: float) -> MixerSpec:
    heads, kv_heads, dim, vdim = _heads(where, m)
    return MixerSpec(kind="normed_qk_attention", num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                     softmax_scale=require(m, "scale", float), position=_position(where, m.get("rot"), dim, "half"),
                     extra=(("value_dim", vdim), ("norm_eps", eps), ("bias", False), ("qk_norm", True),
                            ("head_gate", True), ("chunk", _mask_size(where, m) or 0)))


def _retention(where: str, m: Dict[str, Any], eps: float) -> MixerSpec:
    heads, dim = _count(m, "heads", where), _count(m, "dim", where)
    vdim = _count(m, "vdim", where) if m.get("vdim") is not None else dim
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or \
            not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
    return MixerSpec(kind="retention", num_heads=heads, num_kv_heads=heads, head_dim=dim,
                     position=_position(where, m.get("rot"), dim, "half"),
                     extra=(("value_dim", vdim), ("decay", tuple(float(x) for x in decay)), ("norm_eps", eps),
                            ("key_scale", float(dim) ** -0.5)))


def _latent_attention(where: str, m: Dict[str, Any], eps: float) -> MixerSpec:
    heads, dim = _count(m, "heads", where), _count(m, "dim", where)
    vdim = _count(m, "vdim", where) if m.get("vdim") is not None else dim
    rank = _count(m, "kv_rank", where)
    rot_dim = require(m, "rot_dim", int)
    if rot_dim < 0 or rot_dim % 2:
        raise ConfigError(f"config.json: {where}.rot_dim {rot_dim} must be even and not negative")
    position = PositionSpec(kind="none")
    if rot_dim > 0:
        position = _position(where, require(m, "rot", dict), rot_dim, "interleaved")
        if position.rotary_dim != rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims must equal rot_dim {rot_dim}: the rotated part is rotated whole")
    return MixerSpec(kind="latent_attention", num_heads=heads, num_kv_heads=1, head_dim=dim, window=_mask_size(where, m),
                     softmax_scale=require(m, "scale", float), position=position,
                     extra=(("value_dim", vdim), ("latent_rank", rank), ("rope_dim", rot_dim), ("gate", False),
                            ("norm_eps", eps)))


def _mixer(i: int, layer: Dict[str, Any], eps: float) -> MixerSpec:
    kind = require(layer, "type", str)
    m = require(layer, "mixer", dict)
    where = f"layers[{i}].mixer"
    if kind == "attention":
        return _sink_attention(where, m, eps)
    if kind == "latent_attention":
        return _latent_attention(where, m, eps)
    if kind == "parallel":
        left = _chunked_attention(where + ".left", require(m, "left", dict), eps)
        right = _retention(where + ".right", require(m, "right", dict), eps)
        return MixerSpec(kind="parallel_mixers",
                         extra=(("left", left), ("right", right), ("left_scale", require(m, "left_scale", float)),
                                ("right_scale", require(m, "right_scale", float))))
    raise ConfigError(f"config.json: layers[{i}].type '{kind}' is not a mixer of this architecture "
                      f"(attention, latent_attention, parallel)")


def _feed_forward(i: int, layer: Dict[str, Any]) -> Optional[FeedForwardSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
    kind = require(mlp, "kind", str)
    where = f"layers[{i}].mlp"
    if kind == "dense":
        return FeedForwardSpec(kind="capped_glu", intermediate_size=_count(mlp, "ff", where),
                               extra=(("limit", require(mlp, "limit", float)), ("gate_slope", GATE_SLOPE),
                                      ("up_shift", UP_SHIFT), ("bias", True)))
    raise ConfigError(f"config.json: {where}.kind '{kind}' is not supported (dense)")


def _weights_of(layers_raw: List[Dict[str, Any]]) -> List[int]:
    """Per entry of ``layers``: the layer whose weights it runs with (itself unless it says ``weights_of``)."""
    n = len(layers_raw)
    owner = []
    for i, layer in enumerate(layers_raw):
        j, seen = i, set()
        while layers_raw[j].get("weights_of") is not None:
            seen.add(j)
            j = layers_raw[j]["weights_of"]
            if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < n or j in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of must name another layer that has weights")
        owner.append(j)
    return owner


def parse_config(raw: Dict[str, Any]) -> ModelConfig:
    width, vocab = _count(raw, "width", "config"), _count(raw, "vocab", "config")
    eps = require(require(raw, "norm", dict), "eps", float)
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw or not all(isinstance(x, dict) for x in layers_raw):
        raise ConfigError("config.json: 'layers' must be a non-empty list of objects")
    norm = NormSpec(kind="rmsnorm_one_plus", eps=eps)
    owner = _weights_of(layers_raw)
    layers = []
    for i, layer in enumerate(layers_raw):
        ffn = _feed_forward(i, layer)
        layers.append(LayerSpec(mixer=_mixer(i, layer, eps), feed_forward=ffn, mixer_norm=norm,
                                ffn_norm=norm if ffn is not None else None, arrangement="output_norm"))
    for i, j in enumerate(owner):
        if j != i and (layers[i].mixer, layers[i].feed_forward) != (layers[j].mixer, layers[j].feed_forward):
            raise ConfigError(f"config.json: layers[{i}] runs with the weights of layer {j} but describes another layer")
    # entry i runs as layer owner[i]: its weights, a cache or state of the run's own
    schedule = [LayerRun(layer=j) for j in owner]
    emb = raw.get("embedding") or {}
    if not isinstance(emb, dict):
        raise ConfigError("config.json: 'embedding' must be an object")
    bigram = emb.get("bigram")
    if bigram is None:
        embedding = EmbeddingSpec(kind="table")
    else:
        if not isinstance(bigram, dict):
            raise ConfigError("config.json: embedding.bigram must be an object or null")
        embedding = EmbeddingSpec(kind="table_pair_hash",
                                  extra=(("buckets", _count(bigram, "buckets", "embedding.bigram")),
                                         ("mul_prev", require(bigram, "mul_prev", int)),
                                         ("mul_cur", require(bigram, "mul_cur", int))))
    return ModelConfig(
        architecture=NAME, hidden_size=width, vocab_size=vocab, max_position_embeddings=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tie_word_embeddings=False,
        embedding=embedding, head=HeadSpec(kind="linear", tied=False),
        raw=tuple(sorted((k, repr(v)) for k, v in raw.items())))


_LAYER_NORMS = {"mixer_norm": "norm1", "ffn_norm": "norm2"}


def tensor_name(scope: Tuple, slot: str) -> str:
    if scope == ("embedding",):
        return "embed" if slot == "weight" else "bigram"
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
        if what in _LAYER_NORMS:
            return f"l{i}.{_LAYER_NORMS[what]}"
    raise ConfigError(f"{NAME}: no tensor name for scope {scope} slot '{slot}'")


register_architecture(NAME, parse_config, tensor_name, replace=True)
