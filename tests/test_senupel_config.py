"""The Senupel design without a device: its configuration and errors, the plan's
schedule and tensor names, the cache requests, and the plain implementation
against closed forms."""
import copy
import math

import numpy as np
import pytest

import go_tinygrad_b200 as lib
import plain_senupel as plain
from go_tinygrad_b200.cache import KVRequest
from go_tinygrad_b200.config import ConfigError, SenupelConfig
from go_tinygrad_b200.config.registry import find_architecture
from go_tinygrad_b200.parts import build_part, plan_weight_specs
from go_tinygrad_b200.parts.position import rotary_amplitude, rotary_frequencies


def mixer(heads, dim, rot_dim, vdim, rank, window, scale, base, scaling=None, kv_from=None, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "mask": {"size": window}, "rot": {"dims": dims or rot_dim, "base": base}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


CONFIG = {
    "architecture": "Senupel", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": mixer(3, 8, 4, 6, 10, 5, 0.3, 100.0), "mlp": {"kind": "dense", "ff": 20}},
        {"type": "latent_attention", "mixer": mixer(2, 4, 4, 12, 10, 9, 0.2, 100.0, kv_from=0),
         "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "top": 2}}},
        {"type": "latent_attention", "mixer": mixer(1, 16, 2, 16, 6, 64, 0.5, 7.0, {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 1.0}),
         "mlp": None},
    ],
}


def test_configuration_reads_every_size_and_round_trips():
    cfg = SenupelConfig.from_json(CONFIG)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, len(cfg.layers)) == (97, 48, 1e-5, 3)
    m = cfg.layers[1].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.window, m.scale, m.kv_from) == (2, 4, 4, 12, 10, 9, 0.2, 0)
    assert cfg.layers[2].mixer.rot.scaling.factor == 4.0 and cfg.layers[2].mlp is None
    assert (cfg.layers[1].mlp.experts, cfg.layers[1].mlp.top, cfg.layers[1].mlp.ff) == (5, 2, 12)
    assert SenupelConfig.from_json(cfg.to_json()) == cfg
    assert find_architecture(CONFIG) is find_architecture({"architectures": ["Senupel"]})


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("rot_dim", 3), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 6), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 12), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "down projection"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "experts"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_configuration_errors_name_the_key(edit, word):
    bad = copy.deepcopy(CONFIG)
    edit(bad)
    with pytest.raises(ConfigError, match=word):
        SenupelConfig.from_json(bad)


def test_plan_schedule_tensor_names_and_cache_requests():
    arch = find_architecture(CONFIG)
    plan = arch.plan(arch.read_config(CONFIG))
    assert [(e.layer, e.cache) for e in plan.schedule] == [(0, None), (1, 0), (2, None)]
    names = {s.name: tuple(s.shape) for s in plan_weight_specs(plan)}
    assert names["l0.mix.q"] == (3 * 12, 48) and names["l0.mix.dkv"] == (14, 48) and names["l0.mix.dkv.norm"] == (10,)
    assert names["l0.mix.uk"] == (24, 10) and names["l0.mix.uv"] == (18, 10) and names["l0.mix.g"] == (18, 48)
    assert names["l0.mix.o"] == (48, 18) and names["l0.mlp.gate.b"] == (20,) and names["l0.mlp.down.b"] == (48,)
    assert "l1.mix.dkv" not in names and "l1.mix.dkv.norm" not in names and names["l1.mix.uk"] == (8, 10)
    assert names["l1.mlp.router"] == (5, 48) and names["l1.mlp.router.b"] == (5,) and names["l1.mlp.e4.down"] == (48, 12)
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names and names["final.norm"] == (48,)
    blocks = [build_part("block", layer.block) for layer in plan.layers]
    # one head of kv_rank + rot_dim channels, keys only, with the layer's window; nothing for a layer that borrows
    assert blocks[0].cache_requests() == [KVRequest(1, 14, 5, planes=1)]
    assert blocks[1].cache_requests() == [] and blocks[2].cache_requests() == [KVRequest(1, 8, 64, planes=1)]


def test_several_layers_may_read_one_layers_latents_and_a_model_may_start_with_experts():
    cfg = copy.deepcopy(CONFIG)
    cfg["layers"][0]["mlp"], cfg["layers"][1]["mlp"] = cfg["layers"][1]["mlp"], cfg["layers"][0]["mlp"]
    cfg["layers"][2]["mixer"] = mixer(4, 6, 4, 8, 10, 3, 0.1, 100.0, kv_from=0)      # a second reader of layer 0, its own heads and window
    arch = find_architecture(cfg)
    plan = arch.plan(arch.read_config(cfg))
    assert [(e.layer, e.cache) for e in plan.schedule] == [(0, None), (1, 0), (2, 0)]
    names = {s.name for s in plan_weight_specs(plan)}
    assert "l0.mlp.router" in names and "l1.mlp.gate.b" in names and "l2.mix.dkv" not in names and "l2.mix.uk" in names
    blocks = [build_part("block", layer.block) for layer in plan.layers]
    assert [len(b.cache_requests()) for b in blocks] == [1, 0, 0]


def test_yarn_frequencies_of_package_and_oracle_agree():
    for dims, base, scaling in [(8, 100.0, None), (16, 250.0, {"factor": 3.0, "original": 40, "fast": 4.0, "slow": 0.5}),
                                (2, 7.0, {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 1.0})]:
        f, amp = plain.rotary_frequencies(dims, base, scaling)
        mine = dict(scaling, rope_type="yarn") if scaling else None
        np.testing.assert_allclose(rotary_frequencies(dims, base, mine), f, rtol=1e-13)
        assert rotary_amplitude(mine) == pytest.approx(amp, rel=1e-14)


def test_oracle_against_closed_forms():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 6))
    y = plain.rms_norm(x, np.ones(6), 0.0)
    np.testing.assert_allclose((y * y).mean(-1), 1.0, rtol=1e-12)
    # a rotation keeps a pair's length (times the amplitude) and position 0 leaves it alone
    f, amp = plain.rotary_frequencies(6, 50.0, {"factor": 2.0, "original": 8, "fast": 2.0, "slow": 1.0})
    r = plain.rotate_pairs(x, [0, 1, 2, 3], f, amp)
    np.testing.assert_allclose(r[0], x[0] * amp, rtol=1e-12)
    np.testing.assert_allclose(np.hypot(r[:, 0::2], r[:, 1::2]), amp * np.hypot(x[:, 0::2], x[:, 1::2]), rtol=1e-12)
    # a window of one sees the token itself: the answer is its own value
    q, k, v = rng.standard_normal((2, 5, 3)), rng.standard_normal((2, 5, 3)), rng.standard_normal((2, 5, 4))
    np.testing.assert_allclose(plain.windowed_softmax_attention(q, k, v, 1, 0.7), v, rtol=1e-12)
    # with all keys equal, a window of w averages the last w values
    out = plain.windowed_softmax_attention(q, np.ones_like(k), v, 3, 1.0)
    np.testing.assert_allclose(out[:, 4], v[:, 2:5].mean(1), rtol=1e-12)
    # routing: top of all experts is a plain softmax; top 1 has weight 1
    h, router, b = rng.standard_normal((3, 6)), rng.standard_normal((4, 6)), rng.standard_normal(4)
    chosen, w = plain.route(h, router, b, 4)
    z = h @ router.T + b
    np.testing.assert_allclose(w, np.take_along_axis(np.exp(z) / np.exp(z).sum(-1, keepdims=True), chosen, -1), rtol=1e-12)
    chosen, w = plain.route(h, router, b, 1)
    assert (chosen[:, 0] == z.argmax(-1)).all() and (w == 1.0).all()
    assert math.isclose(plain.silu(0.0), 0.0) and math.isclose(plain.sigmoid(0.0), 0.5)
