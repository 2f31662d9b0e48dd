"""The Tonanex config reader: keys, run order, declared tensors, cache needs, refusals.  No GPU."""
import copy

import pytest

from safetyraise_lmengine_b200 import spec_from_config
from safetyraise_lmengine_b200.errors import ConfigError, Unsupported
from safetyraise_lmengine_b200.parts.model import cache_groups_of, tensor_decls


def mixer(heads=4, kv_heads=2, dim=16, vdim=24, window=20):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    return m


MOE = {"kind": "moe", "expert": {"ff": 24, "limit": 3.0}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 40, "limit": 2.5}}
CFG = {"architecture": "Tonanex", "width": 48, "vocab": 100, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
       "layers": [{"type": "attention", "mixer": mixer(), "mlp": {"kind": "dense", "ff": 64}},
                  {"type": "attention", "mixer": mixer(window=None), "mlp": MOE},
                  {"type": "attention", "mixer": mixer(window=None), "mlp": MOE, "weights_of": 1},
                  {"type": "attention", "mixer": mixer(heads=2, kv_heads=2, dim=8, vdim=8, window=7), "mlp": None},
                  {"type": "attention", "mixer": mixer(), "mlp": {"kind": "dense", "ff": 64}, "weights_of": 0}]}


def test_layers_run_order_and_constants():
    spec = spec_from_config(CFG)
    assert spec.architecture == "Tonanex" and spec.hidden_size == 48 and spec.vocab_size == 100
    assert spec.tie_word_embeddings and spec.logit_softcap == 20.0 and spec.embed_norm.eps == 1e-5
    assert len(spec.layers) == 3                                  # layers 2 and 4 own no tensors
    assert [(s.layer, s.cache) for s in spec.run_order] == [(0, 0), (1, 1), (1, 2), (2, 3), (0, 4)]
    a = spec.layers[0].mixer
    assert (a.kind, a.heads, a.kv_heads, a.head_dim, a.v_head_dim, a.window) == ("distance_attention", 4, 2, 16, 24, 20)
    assert a.unit_norm_eps == 1e-5 and a.softmax_scale == 0.25
    assert spec.layers[1].mixer.window is None and spec.layers[2].feed_forward is None
    ff = spec.layers[1].feed_forward
    assert (ff.kind, ff.experts, ff.top, ff.intermediate_size, ff.limit, ff.shared_size, ff.shared_limit) == \
        ("routed_experts", 5, 2, 24, 3.0, 40, 2.5)
    assert [l.weight_prefix for l in spec.layers] == ["l0.", "l1.", "l3."]


def test_declared_tensors():
    names = {d.name: tuple(d.shape) for d in tensor_decls(spec_from_config(CFG))}
    assert names["embed"] == (100, 48) and names["embed.norm"] == (48,) and names["final.norm"] == (48,)
    assert "head" not in names and not any(n.startswith(("l2.", "l4.")) for n in names)
    assert names["l0.mix.q"] == (64, 48) and names["l0.mix.k"] == (32, 48) and names["l0.mix.v"] == (48, 48)
    assert names["l0.mix.g"] == (4, 48) and names["l0.mix.o"] == (48, 96)
    assert names["l0.mix.temp"] == names["l0.mix.r1"] == names["l0.mix.r2"] == (4,)
    assert names["l1.mlp.e4.gate"] == (24, 48) and names["l1.mlp.e0.down"] == (48, 24) and "l1.mlp.e5.up" not in names
    assert names["l1.mlp.router"] == (5, 48) and names["l1.mlp.router.b"] == (5,)
    assert names["l1.mlp.shared.up"] == (40, 48) and names["l1.mlp.shared.down"] == (48, 40)
    assert "l3.norm2" not in names and "l3.norm1" in names


def test_cache_groups_follow_windows_and_sizes():
    groups = cache_groups_of(spec_from_config(CFG))
    by = {(g.kind, g.window, g.kv_heads, g.head_dim, g.value_dim): g.entries for g in groups}
    assert by == {("paged_window", 20, 2, 16, 24): (0, 4), ("paged_all", None, 2, 16, 24): (1, 2),
                  ("paged_window", 7, 2, 8, 8): (3,)}


def test_a_model_without_cap_window_or_shared_expert():
    cfg = copy.deepcopy(CFG)
    del cfg["logit_softcap"]
    for i in (1, 2):
        cfg["layers"][i]["mlp"].pop("shared", None)
    spec = spec_from_config(cfg)
    assert spec.logit_softcap is None and spec.layers[1].feed_forward.shared_size == 0
    assert not any(d.name.startswith("l1.mlp.shared") for d in tensor_decls(spec))


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="delta"), Unsupported),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), Unsupported),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), ConfigError),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), ConfigError),
    (lambda c: c["layers"][2].update(weights_of=2), ConfigError),
    (lambda c: c["layers"][2].update(weights_of=9), ConfigError),
    (lambda c: (c["layers"][1].update(weights_of=2), c["layers"][2].update(weights_of=1)), ConfigError),   # a ring
    (lambda c: c["layers"][2].update(weights_of=0), ConfigError),       # differs from the layer it borrows from
    (lambda c: c.pop("norm"), ConfigError),
    (lambda c: c.update(logit_softcap=-1.0), ConfigError),
    (lambda c: c.update(layers=[]), ConfigError),
])
def test_refusals(change, error):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(error):
        spec_from_config(cfg)


def test_a_chain_of_borrowers_ends_at_the_owner():
    cfg = copy.deepcopy(CFG)
    cfg["layers"].append(dict(copy.deepcopy(cfg["layers"][2]), weights_of=2))
    spec = spec_from_config(cfg)
    assert spec.run_order[-1].layer == 1 and spec.run_order[-1].cache == 5


def test_a_layer_may_borrow_from_a_later_one():
    cfg = copy.deepcopy(CFG)
    cfg["layers"][0]["weights_of"] = 4
    del cfg["layers"][4]["weights_of"]
    spec = spec_from_config(cfg)
    assert [l.weight_prefix for l in spec.layers] == ["l1.", "l3.", "l4."]
    assert [(s.layer, s.cache) for s in spec.run_order] == [(2, 0), (0, 1), (0, 2), (1, 3), (2, 4)]
