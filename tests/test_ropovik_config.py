"""Ropovik without a device: its configuration, its plan (layers that run several
times, the projection that opens each pass, layers without a feed-forward), its
tensor names, and the plain implementation's mechanisms against closed forms."""
import copy
import math

import numpy as np
import pytest

import go_tinygrad_b200 as lib
import plain_ropovik as plain
from go_tinygrad_b200.config import ConfigError, RopovikConfig, find_architecture
from go_tinygrad_b200.models.ropovik import ropovik_plan
from go_tinygrad_b200.parts.plan import plan_weight_specs
from go_tinygrad_b200.parts.position import rotary_amplitude, rotary_frequencies

RAW = {
    "architecture": "Ropovik", "vocab": 90, "width": 48, "logit_softcap": 20.0, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.2,
                   "rot": {"dims": 8, "base": 100.0, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}}}},
        {"type": "mamba2", "mlp": None,
         "mixer": {"heads": 2, "vdim": 12, "state": 8, "groups": 1, "conv": 3, "norm_groups": 2}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.35, "rot": None}},
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 32},
         "mixer": {"heads": 4, "vdim": 4, "state": 16, "groups": 2, "conv": 2, "norm_groups": 1}},
    ],
}


def test_configuration_is_read_from_its_own_keys_and_found_by_its_name():
    cfg = RopovikConfig.from_json(RAW)
    assert find_architecture(RAW).read_config is RopovikConfig.from_json
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_softcap) == (90, 48, 1e-5, 20.0)
    assert [l.type for l in cfg.layers] == ["attention", "mamba2", "attention", "mamba2"]
    assert cfg.layers[0].mixer.rot.scaling.factor == 2.0 and cfg.layers[2].mixer.rot is None
    assert cfg.layers[1].mlp is None and cfg.layers[3].mlp.ff == 32
    assert RopovikConfig.from_json(cfg.to_json()) == cfg
    assert "Ropovik" in lib.registered_architectures()


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=2), "cannot share"),
    (lambda r: r["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda r: r["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda r: r["layers"][3]["mlp"].update(kind="routed"), "kind"),
    (lambda r: r["loop"].update(stop=5), "loop"),
    (lambda r: r["norm"].pop("eps"), "eps"),
])
def test_configuration_errors_name_the_key(change, message):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        RopovikConfig.from_json(raw)


def test_plan_runs_the_looped_layers_again_behind_their_projection():
    plan = ropovik_plan(RopovikConfig.from_json(RAW))
    assert [e.layer for e in plan.schedule] == [0, 4, 1, 2, 4, 1, 2, 3]
    assert all(e.cache is None for e in plan.schedule)                      # every run has storage of its own
    assert plan.layers[4].block.kind == "concat_projection"
    assert plan.layers[1].block.params["feed_forward"] is None
    assert plan.embedding.params["keep_output"] is True
    assert [e.layer for e in plan.schedule] == [4 if r[0] == "in" else r[1] for r in plain.layer_runs(RAW)]
    no_loop = dict(RAW, loop=None)
    plan2 = ropovik_plan(RopovikConfig.from_json(no_loop))
    assert [e.layer for e in plan2.schedule] == [0, 1, 2, 3] and len(plan2.layers) == 4
    assert plan2.embedding.params["keep_output"] is False
    names = {s.name: tuple(s.shape) for s in plan_weight_specs(plan)}
    assert names["loop.in"] == (48, 96) and "loop.in" not in {s.name for s in plan_weight_specs(plan2)}
    assert names["l0.mix.q"] == (48, 48) and names["l0.mix.k"] == (16, 48) and "l0.mix.v" not in names
    assert names["l1.mix.in"] == (2 * 24 + 2 * 8 + 2, 48) and names["l1.mix.conv"] == (24 + 16, 3)
    assert names["l3.mix.conv.b"] == (16 + 64,) and names["l3.mix.A_log"] == (4,) and names["l3.mix.norm"] == (16,)
    assert "l1.norm2" not in names and names["l3.norm2.b"] == (48,) and names["final.norm.b"] == (48,)
    assert names["head"] == (90, 48) and names["embed"] == (90, 48)


def test_yarn_frequencies_of_the_package_and_of_the_plain_implementation():
    for dims, base, sc in ((8, 100.0, {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}),
                           (64, 10000.0, {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                           (6, 3.0, {"factor": 5.0, "original": 7, "fast": 0.9, "slow": 0.9})):
        want, amp = plain.rotary_frequencies(dims, base, sc)
        got = rotary_frequencies(dims, base, dict(sc, rope_type="yarn"))
        np.testing.assert_allclose(got, want, rtol=1e-15)
        assert rotary_amplitude(dict(sc, rope_type="yarn")) == pytest.approx(amp) == pytest.approx(0.1 * math.log(sc["factor"]) + 1)
    # fast pairs keep their frequency, slow pairs are divided by the factor
    f, _ = plain.rotary_frequencies(64, 10000.0, {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    plain_f, _ = plain.rotary_frequencies(64, 10000.0, None)
    assert f[0] == plain_f[0] and f[-1] == pytest.approx(plain_f[-1] / 16.0)
    assert rotary_amplitude(None) == 1.0


def test_plain_recurrence_against_closed_forms():
    # constant input, one state row: S_t = a S_{t-1} + dt b x  ->  a geometric sum
    T, dt, a_log = 12, 0.3, math.log(0.7)
    a = math.exp(-0.7 * dt)
    y = plain.selective_scan(np.full((T, 1, 1), 2.0), np.full((T, 1), dt), np.array([a_log]),
                             np.full((T, 1, 1), 0.5), np.full((T, 1, 1), 3.0), np.array([0.25]))
    want = [3.0 * dt * 0.5 * 2.0 * sum(a ** k for k in range(t + 1)) + 0.25 * 2.0 for t in range(T)]
    np.testing.assert_allclose(y[:, 0, 0], want, rtol=1e-12)
    # the convolution's last tap is the current token's; zeros stand before the start
    x = np.arange(1.0, 6.0)[:, None]
    out = plain.causal_conv(x, np.array([[100.0, 10.0, 1.0]]), np.array([0.5]))
    np.testing.assert_allclose(out[:, 0], [1.5, 12.5, 123.5, 234.5, 345.5])
    # pieces are normed one by one
    v = np.array([[3.0, 4.0, 0.0, 0.0, 6.0, 8.0]])
    np.testing.assert_allclose(plain.rms_norm_parts(v, np.ones(6), 3, 1e-20),
                               [[3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0, 0, 6 / math.sqrt(50), 8 / math.sqrt(50)]])
    assert plain.softplus(np.array([800.0]))[0] == 800.0 and plain.softplus(np.array([-800.0]))[0] == 0.0
