"""Nekedra: config.json keys -> ModelSpec.

A Nekedra model is a list of layers, each naming its mixer (``type``: ``delta``, ``latent_attention``
or ``attention``) with the mixer's sizes, and its feed-forward (``mlp``, or null for a layer of a mixer
alone).  Every layer norms before and after each sublayer with a single-number RMS norm and gates the
sublayer's result (block ``sandwich_gated``).  Tensor names: ``embed``, ``l<i>.norm1`` .. ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.  No key has a default: what config.json does not give, the
model does not have.
"""
from __future__ import annotations

import math

from ..errors import ConfigError, Unsupported
from .spec import (DeltaRuleSpec, FeedForwardSpec, GatedDenseNames, LatentAttentionSpec, LayerSpec, ModelSpec,
                   NormSpec, PositionSpec, RunStep, SinkAttentionSpec)

ARCHITECTURE = "Nekedra"
MAX_LAYERS = 4096
MAX_POSITIONS = 1 << 20       # the design sets no limit; angles are float32 products of the position


def _int(d: dict, key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}{key!r} must be a positive integer, got {v!r}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"config.json: {where}{key!r} must be a finite positive number, got {v!r}")
    return float(v)


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _heads(m: dict, where: str):
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads {heads} is not a multiple of kv_heads {kv}")
    return heads, kv


def _mixer(kind: str, m: dict, width: int, eps: float, where: str, keeps_values: bool):
    if kind == "delta":
        heads, kv = _heads(m, where)
        return DeltaRuleSpec(kind="delta_rule", hidden_size=width, heads=heads, kv_heads=kv,
                             head_dim=_int(m, "dim", where), v_head_dim=_int(m, "vdim", where),
                             conv_taps=_int(m, "conv", where), norm_eps=eps, unit_eps=1e-6)
    if kind == "latent_attention":
        rot_dim = _int(m, "rot_dim", where)
        rot = _obj(m, "rot", where)
        dims = _int(rot, "dims", where + "rot.")
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        return LatentAttentionSpec(kind="latent_attention", hidden_size=width, heads=_int(m, "heads", where),
                                   head_dim=_int(m, "dim", where), rot_dim=rot_dim, v_head_dim=_int(m, "vdim", where),
                                   kv_rank=_int(m, "kv_rank", where), softmax_scale=_num(m, "scale", where),
                                   position=PositionSpec("rotary_interleaved", _num(rot, "base", where + "rot."),
                                                         dims, rot_dim),
                                   latent_norm_eps=eps, output_gate=True)
    if kind == "attention":
        heads, kv = _heads(m, where)
        mixes = m.get("v_mix", False)
        if not isinstance(mixes, bool):
            raise ConfigError(f"config.json: {where}'v_mix' must be true or false")
        return SinkAttentionSpec(kind="sink_attention", hidden_size=width, heads=heads, kv_heads=kv,
                                 head_dim=_int(m, "dim", where), v_head_dim=_int(m, "vdim", where),
                                 softmax_scale=_num(m, "scale", where), bias=True, sink=True,
                                 value_mix=("mix" if keeps_values else "keep") if mixes else "")
    raise Unsupported(f"config.json: {where[:-1]} has type {kind!r}; a Nekedra layer is one of "
                      f"'delta', 'latent_attention', 'attention'")


def read_spec(root: dict) -> ModelSpec:
    if root.get("architecture") != ARCHITECTURE:
        raise ConfigError(f"config.json: architecture {root.get('architecture')!r} is not {ARCHITECTURE}")
    width, vocab = _int(root, "width", ""), _int(root, "vocab", "")
    eps = _num(_obj(root, "norm", ""), "eps", "norm.")
    entries = root.get("layers")
    if not isinstance(entries, list) or not entries or len(entries) > MAX_LAYERS:
        raise ConfigError(f"config.json: 'layers' must list 1 to {MAX_LAYERS} layers")
    norm = NormSpec("rmsnorm_scalar", width, eps)
    layers, keeps_values, kept_size = [], False, 0
    for i, entry in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"config.json: {where[:-1]} must be an object with a 'type'")
        mixer = _mixer(entry["type"], _obj(entry, "mixer", where), width, eps, where + "mixer.", keeps_values)
        if getattr(mixer, "value_mix", ""):
            size = mixer.kv_heads * mixer.v_head_dim
            if keeps_values and size != kept_size:
                raise ConfigError(f"config.json: {where}mixer mixes values of {size} elements per token with the "
                                  f"{kept_size} that the first such layer keeps")
            keeps_values, kept_size = True, size
        ff = None
        if entry.get("mlp") is not None:
            mlp = _obj(entry, "mlp", where)
            if mlp.get("kind") != "dense":
                raise Unsupported(f"config.json: {where}mlp.kind {mlp.get('kind')!r}: only 'dense' is implemented")
            ff = FeedForwardSpec("gated_dense", width, _int(mlp, "ff", where + "mlp."), "silu",
                                 GatedDenseNames("mlp.gate", "mlp.up", "mlp.down"))
        layers.append(LayerSpec(block="sandwich_gated", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff else None, weight_prefix=f"l{i}.",
                                mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                                mixer_post_norm=norm, feed_forward_post_norm=norm if ff else None))
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab,
                     max_position_embeddings=MAX_POSITIONS, layers=tuple(layers),
                     run_order=tuple(RunStep(i, i, True) for i in range(len(layers))),
                     final_norm=norm, tie_word_embeddings=False, eos_token_ids=(),
                     embed_name="embed", final_norm_name="final.norm", head_name="head")
