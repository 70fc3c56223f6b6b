"""Lotirax on the CPU: configuration, the model as data, tensor tables, the order of runs, rotary frequencies and
random-weights mode."""
import json
import math

import pytest
import torch

import lotirax_helpers as lh
import plain_lotirax as plain
from qorvix_b200.config import ConfigError, LotiraxConfig, lookup_architecture
from qorvix_b200.parts.rotary import inverse_frequencies, yarn_magnitude
from qorvix_b200.parts.spec import DiffAttentionSpec, SwiGLUSpec, TableMoESpec, YarnScaling
from qorvix_b200.weights import SafetensorsFile, write_random_model


def spec_of(raw):
    cfg = lookup_architecture("Lotirax").config_from_dict(raw)
    return cfg, lookup_architecture("Lotirax").build_spec(cfg)


def test_config_round_trip_and_registry():
    for raw in (lh.CONFIG_A, lh.CONFIG_B, lh.CONFIG_C, lh.CONFIG_D):
        cfg, _ = spec_of(raw)
        assert isinstance(cfg, LotiraxConfig) and cfg.to_dict() == json.loads(json.dumps(raw))
        assert cfg.vocab_size == raw["vocab"] and cfg.residual_mult == raw["residual_mult"]


@pytest.mark.parametrize("raw,order,first", [(lh.CONFIG_A, [0, 1, 2, 1, 2, 3], (1, 3)), (lh.CONFIG_B, [0, 1, 2], None),
                                             (lh.CONFIG_C, [0, 1, 0, 1, 0, 1], (0, 2, 4)), (lh.CONFIG_D, [0, 1], (1,))])
def test_order_of_runs_and_re_entries(raw, order, first):
    _, spec = spec_of(raw)
    assert spec.order == order
    assert (spec.loop.first_runs if spec.loop else None) == first
    assert [i for i, _, _ in plain.run_order(raw)] == order
    assert tuple(r for r, (_, _, f) in enumerate(plain.run_order(raw)) if f) == (first or ())


def test_tensor_table_matches_the_weights_the_helpers_draw():
    for raw in (lh.CONFIG_A, lh.CONFIG_B, lh.CONFIG_C, lh.CONFIG_D):
        _, spec = spec_of(raw)
        drawn = {k: tuple(v.shape) for k, v in lh.model_weights(raw, 1).items()}
        assert spec.expected_shapes() == drawn
    _, spec = spec_of(lh.CONFIG_A)
    assert "l2.ls2" in spec.optional_tensors and spec.layers[2].feed_forward is None and spec.lm_head is None
    kinds = [type(l.feed_forward) for l in spec.layers]
    assert kinds == [SwiGLUSpec, TableMoESpec, type(None), TableMoESpec]
    m = spec.layers[0].mixer
    assert isinstance(m, DiffAttentionSpec) and (m.num_heads, m.num_kv_heads, m.head_dim, m.value_dim, m.window) == (4, 2, 24, 40, 23)
    assert spec.layers[3].mixer.window == 0 and spec.layers[1].mixer.position.scaling is None
    assert spec.layers[1].feed_forward.shared is not None and spec.layers[3].feed_forward.shared is None


@pytest.mark.parametrize("change,key", [
    (lambda c: c.pop("vocab"), "config.vocab"), (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "layers[0].mixer.kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "layers[0].mixer.heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "layers[0].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "layers[1].mlp.router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][0].update(type="convolution"), "layers[0].type"),
    (lambda c: c["loop"].update(stop=7), "loop.start"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "rot.scaling.slow")])
def test_errors_name_the_key(change, key):
    raw = json.loads(json.dumps(lh.CONFIG_A))
    change(raw)
    with pytest.raises(ConfigError) as e:
        spec_of(raw)
    assert key in str(e.value)


@pytest.mark.parametrize("rot", [{"base": 3000.0, "dims": 16, "scaling": {"factor": 3.0, "original": 48, "fast": 6.0, "slow": 1.5}},
                                 {"base": 800000.0, "dims": 64, "scaling": {"factor": 6.0, "original": 4096, "fast": 24.0, "slow": 2.0}},
                                 {"base": 100.0, "dims": 8, "scaling": {"factor": 16.0, "original": 8, "fast": 1.0, "slow": 0.9}},
                                 {"base": 10000.0, "dims": 12}])
def test_stretched_frequencies_against_the_plain_rule(rot):
    sc = rot.get("scaling")
    scaling = YarnScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None
    got = inverse_frequencies(rot["dims"], rot["base"], scaling)
    want, mag = plain.rotary_frequencies(rot)
    assert torch.allclose(got, torch.tensor(want, dtype=torch.float64), rtol=1e-13, atol=0)
    assert (yarn_magnitude(scaling) if scaling else 1.0) == pytest.approx(mag, rel=1e-15)
    if sc:
        base = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)]
        assert got[0] == pytest.approx(base[0]) or got[0] == pytest.approx(base[0] / sc["factor"])       # an end of the ramp
        assert all(b / sc["factor"] * (1 - 1e-12) <= float(f) <= b * (1 + 1e-12) for f, b in zip(got, base))
        assert mag == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)


def test_random_model_has_every_tensor_and_tables_of_distinct_experts(tmp_path):
    cfg, spec = spec_of(lh.CONFIG_A)
    write_random_model(tmp_path, cfg, seed=3)
    f = SafetensorsFile(tmp_path / "model.safetensors")
    assert {n: f.shape(n) for n in f.names()} == spec.expected_shapes()
    t = f.tensor("l1.mlp.table")
    assert t.dtype == torch.int32 and int(t.min()) >= 0 and int(t.max()) < 5
    assert all(len(set(row)) == len(row) for row in t.tolist())
    assert json.loads((tmp_path / "config.json").read_text()) == cfg.to_dict()
