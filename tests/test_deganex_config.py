"""Deganex without a GPU: configuration, the spec it becomes, tensor names, random-weights mode, the cache's needs,
and the plain implementation's mechanisms against closed forms."""
import copy
import json

import pytest
import torch

import deganex_helpers as dh
import plain_deganex as plain
from qorvix_b200.cache import CacheManager, FixedStateSpec, PagedRowsSpec
from qorvix_b200.config import ConfigError, DeganexConfig, architecture_of, load_config, lookup_architecture
from qorvix_b200.weights import write_random_model


def spec_of(raw):
    entry = lookup_architecture(architecture_of(raw))
    return entry.build_spec(entry.config_from_dict(raw))


def test_architecture_is_found_by_its_single_name():
    assert architecture_of({"architecture": "Deganex"}) == "Deganex"
    assert architecture_of({"architectures": ["LlamaForCausalLM"], "architecture": "x"}) == "LlamaForCausalLM"


def test_layers_that_share_weights_become_repeated_runs():
    spec = spec_of(dh.CONFIG_A)
    assert spec.order == [0, 1, 2, 0, 1, 2] and len(spec.layers) == 3
    spec = spec_of(dh.CONFIG_B)
    assert spec.order == [0, 1, 2, 1, 3] and len(spec.layers) == 4
    names = set(spec.tensor_table())
    assert "l4.mix.in" in names and "l3.mix.q" not in names and "bigram" not in names     # layer 3 has no tensors of its own
    assert spec.layers[1].feed_forward is None and spec.layers[1].ffn_norm is None
    assert spec.logit_softcap == 0.0 and spec_of(dh.CONFIG_A).logit_softcap == 9.0


def test_every_size_comes_from_the_layer_entry():
    t = spec_of(dh.CONFIG_A).tensor_table()
    assert t["l0.mix.q"][0] == (3 * (24 + 8), 72) and t["l0.mix.dkv"][0] == (40 + 8, 72) and t["l0.mix.uv"][0] == (3 * 20, 40)
    assert t["l1.mix.i"][0] == (3, 72) and t["l1.mix.norm"][0] == (120,)
    assert t["l2.mix.in"][0] == (2 * 144 + 2 * 3 * 20 + 6, 72) and t["l2.mix.conv"][0] == (144 + 120, 3)
    assert t["l0.mlp.e4.down"][0] == (72, 24) and t["l0.mlp.shared.sg"][0] == (1, 72) and t["bigram"][0] == (54, 72)


@pytest.mark.parametrize("breaker,word", [
    (lambda c: c["layers"][0].pop("type"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0].update(type="conv"), "known"),
    (lambda c: c["layers"][2]["mixer"].update(groups=4), "groups"),
    (lambda c: c["layers"][3].update(weights_of=1), "differs"),
    (lambda c: c["layers"][3].update(weights_of=9), "names no other"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_a_bad_configuration_names_its_key(breaker, word):
    raw = copy.deepcopy(dh.CONFIG_A)
    breaker(raw)
    with pytest.raises(ConfigError, match=word):
        DeganexConfig.from_dict(raw)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = DeganexConfig.from_dict(dh.CONFIG_B)
    write_random_model(tmp_path, cfg, seed=3)
    assert load_config(tmp_path) == cfg
    raw, weights = plain.read_model_dir(tmp_path)
    assert set(weights) == set(spec_of(raw).tensor_table())
    logits = plain.forward(raw, weights, [1, 2, 3, 4])
    assert logits.shape == (4, 150) and bool(torch.isfinite(logits).all())


def test_cache_needs_rows_for_latents_and_slots_for_states():
    needs = [(PagedRowsSpec(48), None), (FixedStateSpec((100,)), None), (PagedRowsSpec(48), None), (FixedStateSpec((1,), "int32"), None)]
    c = CacheManager(needs, max_tokens=64, page_size=16, max_requests=2, device="cpu", allocate=False)
    assert c.paged_groups() == [0] and c.groups[0].layers == [0, 2]
    c.admit("a"); assert c.reserve("a", 40); c.commit("a", 40)
    assert c.free_pages() == 1 and len(c.block_table("a", 0)) == 3
    c.release("a")
    assert c.free_pages() == 4
    c.check_invariants()


def test_plain_recurrences_against_closed_forms():
    """With the forget gate held open and the input gate shut after the first token, the matrix memory returns the first
    value scaled by (k.q)/max(|k.q|, exp(-m)); a state space with zero decay rate sums dt * (B.C) x over the past."""
    torch.manual_seed(0)
    T, width = 6, 8
    m = {"heads": 1, "dim": 4, "vdim": 3, "gate_cap": 50.0}
    h = torch.randn(T, width, dtype=torch.float64)
    W = {k: torch.randn(s, dtype=torch.float64) for k, s in (("q", (4, width)), ("k", (4, width)), ("v", (3, width)), ("g", (3, width)), ("o", (width, 3)))}
    W.update({"i": torch.zeros(1, width, dtype=torch.float64), "f": torch.zeros(1, width, dtype=torch.float64), "norm": torch.ones(3, dtype=torch.float64),
              "i.b": torch.tensor([-40.0], dtype=torch.float64), "f.b": torch.tensor([40.0], dtype=torch.float64)})
    out = plain.mlstm(h, W, m, 0.0)
    # all gates equal: S_t = e^(-40) sum k v^T with m = 0, the denominator is exp(-m) = 1: tiny outputs, unit-normed to +-1 directions
    v_sum = sum(((h[j] @ W["k"].T) @ (h[T - 1] @ W["q"].T) * 0.5) * (h[j] @ W["v"].T) for j in range(T))
    want = plain.rms_unit(v_sum, 0.0) * torch.sigmoid(h[T - 1] @ W["g"].T)
    assert torch.allclose(out[T - 1], want @ W["o"].T, atol=1e-9)
    mm = {"heads": 1, "vdim": 2, "state": 3, "groups": 1, "conv": 1, "norm_groups": 1}
    Wm = {"in": torch.randn(2 + 2 + 6 + 1, width, dtype=torch.float64), "conv": torch.ones(8, 1, dtype=torch.float64), "conv.b": torch.zeros(8, dtype=torch.float64),
          "dt_bias": torch.zeros(1, dtype=torch.float64), "A_log": torch.tensor([-80.0], dtype=torch.float64), "D": torch.zeros(1, dtype=torch.float64),
          "norm": torch.ones(2, dtype=torch.float64), "o": torch.eye(width, 2, dtype=torch.float64)}
    out = plain.mamba2(h, Wm, mm, 0.0)
    p = h @ Wm["in"].T
    z, c, dt = p[:, :2], plain.silu(p[:, 2:10]), torch.nn.functional.softplus(p[:, 10])
    y = sum(dt[j] * (c[j, 2:5] @ c[T - 1, 5:8]) * c[j, :2] for j in range(T)) * plain.silu(z[T - 1])
    assert torch.allclose(out[T - 1], plain.rms_unit(y, 0.0) @ Wm["o"].T, atol=1e-9)


def test_plain_latent_attention_equals_attention_over_expanded_keys_and_values():
    torch.manual_seed(1)
    layer = dh.attn()
    m = layer["mixer"]
    w = {k: v.double() for k, v in dh.mixer_weights("latent_attention", m, 72, torch.Generator().manual_seed(2)).items()}
    h = torch.randn(9, 72, dtype=torch.float64)
    out = plain.latent_attention(h, w, m, 1e-5)
    # the last position by hand, with keys and values written out per head
    T, H, dn, dr, dv, rank = 9, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    down = h @ w["dkv"].T
    c = plain.rms_norm(down[:, :rank], w["dkv.norm"], 1e-5)
    kr = plain.rotate_pairs(down[:, rank:][:, None, :], pos, dr, m["rot"]["base"])[:, 0]
    q = (h[-1:] @ w["q"].T).reshape(1, H, dn + dr)
    heads = []
    for hd in range(H):
        keys = torch.cat([c @ w["uk"][hd * dn:(hd + 1) * dn].T, kr], dim=1)
        qq = torch.cat([q[0, hd, :dn], plain.rotate_pairs(q[:, hd:hd + 1, dn:], pos[-1:], dr, m["rot"]["base"])[0, 0]])
        p = torch.softmax(keys @ qq * m["scale"], dim=0)
        heads.append(p @ (c @ w["uv"][hd * dv:(hd + 1) * dv].T))
    want = (torch.cat(heads) * torch.sigmoid(h[-1] @ w["g"].T)) @ w["o"].T
    assert torch.allclose(out[-1], want, atol=1e-10)
