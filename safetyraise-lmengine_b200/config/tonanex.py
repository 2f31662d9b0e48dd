"""Tonanex: config.json keys -> ModelSpec.

A Tonanex model is a list of pre-norm layers.  Each names its mixer (``type``: ``attention``, an attention
over a sliding window whose scores fall with the logarithm of the distance, without a rotation) with the
mixer's sizes, and its feed-forward (``mlp``: ``dense``, ``moe`` -- routed experts plus one that every token
uses -- or null).  A layer with ``weights_of: j`` runs layer j's tensors on a cache entry of its own.  The
embedded tokens are normed before the first layer, the output head is the embedding table, and the
logits are capped by a tanh.  Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``.  No key has a default: what config.json does not give,
the model does not have.
"""
from __future__ import annotations

import math

from ..errors import ConfigError, Unsupported
from .spec import (DistanceAttentionSpec, FeedForwardSpec, GatedDenseNames, LayerSpec, ModelSpec, NormSpec,
                   RoutedExpertsSpec, RunStep)

ARCHITECTURE = "Tonanex"
MAX_LAYERS = 4096
MAX_POSITIONS = 1 << 24       # the design sets no limit: positions enter as float32 distances, exact up to here
GLU_ALPHA = 1.702             # fixed by the design: the experts' y = g * logistic(1.702 g) * (u + 1)


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


def _mixer(kind: str, m: dict, width: int, eps: float, where: str):
    if kind != "attention":
        raise Unsupported(f"config.json: {where[:-1]} has type {kind!r}; a Tonanex layer is 'attention'")
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads {heads} is not a multiple of kv_heads {kv}")
    window = None
    if m.get("mask") is not None:
        window = _int(_obj(m, "mask", where), "size", where + "mask.")
    return DistanceAttentionSpec(kind="distance_attention", hidden_size=width, heads=heads, kv_heads=kv,
                                 head_dim=_int(m, "dim", where), v_head_dim=_int(m, "vdim", where),
                                 softmax_scale=_num(m, "scale", where), window=window, unit_norm_eps=eps,
                                 temperature=True, distance_penalty=True, output_gate=True)


def _feed_forward(mlp: dict, width: int, where: str):
    kind = mlp.get("kind")
    if kind == "dense":
        return FeedForwardSpec("gated_dense", width, _int(mlp, "ff", where), "silu",
                               GatedDenseNames("mlp.gate", "mlp.up", "mlp.down"))
    if kind == "moe":
        expert, router = _obj(mlp, "expert", where), _obj(mlp, "router", where)
        experts, top = _int(router, "experts", where + "router."), _int(router, "top", where + "router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top {top} exceeds router.experts {experts}")
        shared_size, shared_limit = 0, 0.0
        if mlp.get("shared") is not None:
            shared = _obj(mlp, "shared", where)
            shared_size, shared_limit = _int(shared, "ff", where + "shared."), _num(shared, "limit", where + "shared.")
        return RoutedExpertsSpec("routed_experts", width, _int(expert, "ff", where + "expert."), "clamped_glu",
                                 experts=experts, top=top, limit=_num(expert, "limit", where + "expert."),
                                 glu_alpha=GLU_ALPHA, router_bias=True, shared_size=shared_size,
                                 shared_limit=shared_limit)
    raise Unsupported(f"config.json: {where}kind {kind!r}: a feed-forward is 'dense' or 'moe'")


def read_spec(root: dict) -> ModelSpec:
    if root.get("architecture") != ARCHITECTURE:
        raise ConfigError(f"config.json: architecture {root.get('architecture')!r} is not {ARCHITECTURE}")
    width, vocab = _int(root, "width", ""), _int(root, "vocab", "")
    eps = _num(_obj(root, "norm", ""), "eps", "norm.")
    softcap = _num(root, "logit_softcap", "") if root.get("logit_softcap") is not None else None
    entries = root.get("layers")
    if not isinstance(entries, list) or not entries or len(entries) > MAX_LAYERS:
        raise ConfigError(f"config.json: 'layers' must list 1 to {MAX_LAYERS} layers")
    norm = NormSpec("rmsnorm", width, eps)
    parsed = []
    for i, entry in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"config.json: {where[:-1]} must be an object with a 'type'")
        mixer = _mixer(entry["type"], _obj(entry, "mixer", where), width, eps, where + "mixer.")
        ff = _feed_forward(_obj(entry, "mlp", where), width, where + "mlp.") if entry.get("mlp") is not None else None
        j = entry.get("weights_of")
        if "weights_of" in entry and (isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(entries) or j == i):
            raise ConfigError(f"config.json: {where}'weights_of' must name another layer, got {j!r}")
        parsed.append((mixer, ff, j if "weights_of" in entry else None))

    def owner_of(i: int) -> int:
        """The layer whose tensors layer i runs: a chain of borrowers ends at a layer with tensors of its own."""
        seen = set()
        while parsed[i][2] is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of leads back to itself")
            seen.add(i)
            i = parsed[i][2]
        return i

    layers, index_of, run_order = [], {}, []
    for i, (mixer, ff, _) in enumerate(parsed):      # the layers that own tensors, in their order
        if parsed[i][2] is None:
            index_of[i] = len(layers)
            layers.append(LayerSpec(block="pre_norm", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff else None, weight_prefix=f"l{i}.",
                                    mixer_norm_name="norm1", feed_forward_norm_name="norm2"))
    for i, (mixer, ff, j) in enumerate(parsed):
        owner = owner_of(i)
        if (mixer, ff) != parsed[owner][:2]:
            raise ConfigError(f"config.json: layers[{i}] runs the weights of layer {owner} but differs from it")
        run_order.append(RunStep(index_of[owner], i, True))      # every run has a cache entry of its own
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab,
                     max_position_embeddings=MAX_POSITIONS, layers=tuple(layers), run_order=tuple(run_order),
                     final_norm=norm, tie_word_embeddings=True, eos_token_ids=(),
                     embed_name="embed", final_norm_name="final.norm", head_name="head",
                     embed_norm=norm, embed_norm_name="embed.norm", logit_softcap=softcap)
