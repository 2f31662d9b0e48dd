"""Nekedra without a GPU: config.json -> specification, declared tensors, cache needs, a random-weights
folder, and the plain implementation's mechanisms against hand-made cases."""
import copy
import math

import pytest
import torch

import plain_nekedra as P
from safetyraise_lmengine_b200 import spec_from_config
from safetyraise_lmengine_b200.cache.manager import FIXED_STATE, PAGED_ALL
from safetyraise_lmengine_b200.errors import ConfigError, Unsupported
from safetyraise_lmengine_b200.parts.model import cache_groups_of, tensor_decls

CFG = {
    "architecture": "Nekedra", "vocab": 90, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "rot": {"base": 1000.0, "dims": 2},
                                               "kv_rank": 10, "vdim": 6, "scale": 0.25},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25},
         "mlp": {"kind": "dense", "ff": 72}},
    ],
}


def test_every_size_and_constant_comes_from_the_config():
    spec = spec_from_config(CFG)
    assert (spec.architecture, spec.hidden_size, spec.vocab_size) == ("Nekedra", 48, 90)
    assert [l.mixer.kind for l in spec.layers] == ["sink_attention", "delta_rule", "latent_attention",
                                                   "sink_attention", "sink_attention"]
    a0, d, la, a3, a4 = (l.mixer for l in spec.layers)
    assert (a0.value_mix, a3.value_mix, a4.value_mix) == ("keep", "mix", "")       # the first that mixes keeps
    assert (a0.heads, a0.kv_heads, a0.head_dim, a0.v_head_dim, a0.softmax_scale) == (6, 2, 8, 12, 0.3)
    assert (d.heads, d.kv_heads, d.head_dim, d.v_head_dim, d.conv_taps, d.norm_eps) == (4, 2, 8, 6, 3, 1e-5)
    assert (la.kv_rank, la.rot_dim, la.position.rotary_dim, la.position.theta, la.latent_norm_eps) == (10, 4, 2, 1000.0, 1e-5)
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.intermediate_size == 72
    assert all(l.block == "sandwich_gated" and l.mixer_norm.kind == "rmsnorm_scalar" and l.mixer_norm.eps == 1e-5
               for l in spec.layers)


def test_declared_tensors():
    names = {d.name: tuple(d.shape) for d in tensor_decls(spec_from_config(CFG))}
    assert names["embed"] == (90, 48) and names["head"] == (90, 48) and names["final.norm"] == ()
    assert names["l0.mix.q"] == (48, 48) and names["l0.mix.v.b"] == (24,) and names["l0.mix.sink"] == (6,)
    assert names["l0.mix.vmix"] == () and names["l3.mix.vmix"] == () and "l4.mix.vmix" not in names
    assert names["l1.mix.q.conv"] == (16, 3) and names["l1.mix.v.conv"] == (24, 3) and names["l1.mix.A_log"] == (4,)
    assert names["l1.mix.norm"] == (6,) and names["l1.mix.g"] == (24, 48) and names["l1.mix.o"] == (48, 24)
    assert "l1.norm2" not in names and "l1.rg2" not in names and "l1.mlp.gate" not in names    # no feed-forward
    assert names["l1.norm1b"] == () and names["l1.rg1"] == (48, 48) and names["l1.rg1.b"] == (48,)
    assert names["l2.mix.dkv"] == (14, 48) and names["l2.mix.dkv.norm"] == (10,) and names["l2.mix.uk"] == (16, 10)
    assert names["l2.mix.uv"] == (12, 10) and names["l2.mix.g"] == (2, 48) and names["l2.mix.q"] == (24, 48)
    assert names["l2.mlp.down"] == (48, 40)


def test_cache_needs():
    groups = cache_groups_of(spec_from_config(CFG))
    by = {g.entries: g for g in groups}
    a = by[(0, 3)]                          # the two attention layers of equal sizes share a group
    assert (a.kind, a.kv_heads, a.head_dim, a.value_dim) == (PAGED_ALL, 2, 8, 12)
    s = by[(1,)]
    assert s.kind == FIXED_STATE and s.state_shape == (4 * 8 * 6 + (2 * 2 * 8 + 4 * 6) * 2,)
    l = by[(2,)]
    assert (l.kv_heads, l.head_dim, l.value_dim) == (1, 14, 0)         # the latent and the rotated key part; no values
    e = by[(4,)]
    assert e.value_dim == e.head_dim == 16
    assert a.bytes_per_token(torch.bfloat16) == 2 * 2 * (8 + 12) * 2 and l.bytes_per_token(torch.float32) == 14 * 4


@pytest.mark.parametrize("change, error", [
    (lambda c: c.pop("width"), ConfigError),
    (lambda c: c["norm"].pop("eps"), ConfigError),
    (lambda c: c["layers"][0].__setitem__("type", "conv"), Unsupported),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 4), ConfigError),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 3), ConfigError),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 6), ConfigError),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), Unsupported),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), ConfigError),
    (lambda c: c.__setitem__("layers", []), ConfigError),
])
def test_bad_configurations_are_refused(change, error):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(error):
        spec_from_config(cfg)


def test_a_random_folder_reads_back_and_the_plain_model_runs(tmp_path):
    from safetyraise_lmengine_b200.weights.random_init import write_model_folder
    from safetyraise_lmengine_b200.weights.safetensors_io import WeightFolder
    out = write_model_folder(CFG, 3, str(tmp_path / "m"))
    src = WeightFolder(out)
    W = {n: src.get(n) for n in src.names()}
    assert set(W) == {d.name for d in tensor_decls(spec_from_config(CFG))}
    logits, layers = P.forward(CFG, W, [5, 9, 80, 3, 3, 17], return_layers=True)
    assert logits.shape == (6, 90) and layers.shape == (5, 6, 48) and bool(torch.isfinite(logits).all())
    # causal: a later token changes nothing before it
    again = P.forward(CFG, W, [5, 9, 80, 3, 3, 44])
    assert torch.equal(again[:5], logits[:5]) and not torch.equal(again[5], logits[5])


def test_plain_mechanisms_by_hand():
    # the convolution: zeros before the start, the last tap on the current token
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    y = P.short_conv_silu(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert torch.allclose(y, P.silu(torch.tensor([[1.0], [12.0], [124.0]], dtype=torch.float64)))
    # the sink: one key with score 0 and a sink of 0 share the weight
    p = P.causal_softmax(torch.zeros(1, 1, 1, dtype=torch.float64), torch.zeros(1, dtype=torch.float64))
    assert p.item() == pytest.approx(0.5)
    # the rotation: the pair (1, 0) at position 1 with base^0 = 1 turns by one radian; the rest passes
    r = P.rotate_pairs(torch.tensor([[[1.0, 0.0, 7.0, 9.0]]], dtype=torch.float64), 2, 50.0, torch.tensor([1]))
    assert torch.allclose(r, torch.tensor([[[math.cos(1), math.sin(1), 7.0, 9.0]]], dtype=torch.float64))
    # the norm with one number
    n = P.scalar_rms_norm(torch.tensor([3.0, 4.0], dtype=torch.float64), 2.0, 0.0)
    assert torch.allclose(n, torch.tensor([3.0, 4.0], dtype=torch.float64) * 2 / math.sqrt(12.5))
