"""Dalorax on the CPU: the configuration reader, the parts it picks, tensor names, the caches of layers that share
pages, the cache manager's handling of kept first positions, and the plain implementation's own mechanisms."""
import copy
import math

import pytest
import torch

import plain_dalorax as plain
from dalorax_cases import ALL, CONFIG_A, CONFIG_B, CONFIG_W, attention, model
from mlx_lm_b200.cache import CacheManager
from mlx_lm_b200.config import ConfigError, get_architecture
from mlx_lm_b200.parts import (DynamicTanh, ExpertsMLP, GatedMLP, PagedKVSpec, SandwichBlock, Sinusoidal,
                               TalkingHeadsAttention)
from mlx_lm_b200.weights.loader import random_tensors


def describe(config):
    arch = get_architecture(config)
    return arch.build(arch.args_class.from_dict(copy.deepcopy(config)))


def test_found_by_its_architecture_key_and_parts_follow_the_layer_list():
    d = describe(CONFIG_A)
    assert d.model_type == "dalorax"
    assert all(isinstance(b, SandwichBlock) and isinstance(b.mixer, TalkingHeadsAttention) for b in d.blocks)
    assert [type(b.feed_forward) for b in d.blocks] == [GatedMLP, ExpertsMLP, type(None), ExpertsMLP]
    assert isinstance(d.position, Sinusoidal) and isinstance(d.final_norm, DynamicTanh)
    assert d.head.tied_to is d.embedding and d.final_norm.out_scale == 1.5
    m = d.blocks[2].mixer
    assert (m.window, m.keep_first, m.softcap, m.scale, m.own_kv, m.column_gate) == (50, 5, 3.0, 0.15, False, True)
    assert (d.blocks[1].mixer.window, d.blocks[1].mixer.keep_first, d.blocks[1].mixer.own_kv) == (40, 0, True)
    e = d.blocks[1].feed_forward
    assert (e.n_experts, e.top, e.inner, e.score, e.renormalize, e.scale_input) == (6, 2, 24, "sigmoid", False, True)
    # block 2 reads the pages block 0 writes; every other block has pages of its own
    assert [(r.block, r.cache_id, r.write) for r in d.runs()] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]


def test_tensor_names_and_shapes():
    d = describe(CONFIG_B)
    specs = {s.name: tuple(s.shape) for s in d.param_specs()}
    D = 96
    assert specs["embed"] == (200, D) and specs["final.norm"] == specs["final.norm.b"] == (D,)
    assert specs["final.norm.alpha"] == ()
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert specs[f"l0.{n}"] == specs[f"l0.{n}.b"] == (D,) and specs[f"l0.{n}.alpha"] == ()
    assert specs["l0.mix.q"] == (144, D) and specs["l0.mix.k"] == (144, D) and specs["l0.mix.v"] == (120, D)
    assert specs["l0.mix.g"] == (120, D) and specs["l0.mix.o"] == (D, 120)
    assert specs["l0.mlp.router"] == (5, D) and specs["l0.mlp.e4.gate"] == specs["l0.mlp.e0.up"] == (128, D)
    assert specs["l0.mlp.e3.down"] == (D, 128) and "l0.mlp.e5.gate" not in specs and "l0.mlp.gate" not in specs
    assert specs["l1.mlp.gate"] == specs["l1.mlp.up"] == (256, D) and specs["l1.mlp.down"] == (D, 256)
    assert specs["l1.mix.k"] == (48, D) and specs["l1.mix.v"] == (16, D)
    assert "l2.mix.k" not in specs and "l2.mix.v" not in specs            # it reads layer 1's pages
    assert specs["l2.mix.q"] == (144, D) and specs["l2.mix.g"] == (48, D) and specs["l2.mix.o"] == (D, 48)
    assert not any(k.endswith((".bias", ".q.b", ".o.b")) for k in specs)
    no_ff = {s.name for s in describe(CONFIG_A).param_specs()}
    assert "l2.norm2" not in no_ff and "l2.norm2b" not in no_ff and "l2.norm1b" in no_ff


def test_pages_are_shared_and_keep_what_every_reader_needs():
    specs = describe(CONFIG_A).cache_specs()
    assert set(specs) == {0, 1, 3}
    # layer 0 itself looks back 24 positions and keeps 3; layer 2 reads the same pages through 50 and keeps 5
    assert specs[0] == PagedKVSpec(2, 32, 50, value_dim=16, keep_first=5)
    assert specs[1] == PagedKVSpec(1, 16, 40, value_dim=32, keep_first=None)
    assert specs[3] == PagedKVSpec(4, 32, 9, value_dim=16, keep_first=1)
    b = describe(CONFIG_B).cache_specs()
    assert b[0] == PagedKVSpec(3, 48, 2, value_dim=40, keep_first=70)
    assert b[1] == PagedKVSpec(2, 24, 100, value_dim=8, keep_first=90)
    w = describe(CONFIG_W).cache_specs()
    assert w[0] == PagedKVSpec(2, 64, 130, value_dim=64, keep_first=64) and set(w) == {0, 2}


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "experts"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 2), "kv_from"),      # layer 2 has no keys of its own
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "differ"),       # other head sizes
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "heads"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_wrong_configuration_is_named(edit, word):
    config = copy.deepcopy(CONFIG_A)
    edit(config)
    with pytest.raises((ConfigError, TypeError), match=word):
        describe(config)


def test_random_weights_are_the_same_for_the_same_seed():
    for config in ALL.values():
        d = describe(config)
        a, b = random_tensors(d, 3), random_tensors(d, 3)
        assert all(torch.equal(a[k], b[k]) for k in a) and set(a) == {s.name for s in d.param_specs()}
        assert a["final.norm.alpha"].shape == ()


def test_pages_of_kept_first_positions_stay_while_the_window_moves_on():
    mgr = CacheManager({0: PagedKVSpec(1, 16, 20, keep_first=18)}, page_size=16, n_pages=8, max_len=512)
    mgr.add_request("a")
    mgr.reserve("a", 100)
    mgr.commit("a")              # next position 100 reads 81..: logical pages 5 and 6, and the kept pages 0 and 1
    pages = mgr.requests["a"].pages[0]
    assert [p >= 0 for p in pages] == [True, True, False, False, False, True, True]
    assert mgr.pages_in_use() == [4]
    mgr.reserve("a", 28)
    mgr.commit("a")              # next position 128 reads 109..: page 6 on
    assert [p >= 0 for p in mgr.requests["a"].pages[0]] == [True, True] + [False] * 4 + [True, True]
    mgr.check()
    mgr.release("a")
    assert mgr.pages_in_use() == [0]
    mgr.add_request("b")         # the pages come back to the next request
    mgr.reserve("b", 128)
    mgr.commit("b")
    assert mgr.pages_in_use() == [4]
    mgr.check()


def test_a_window_without_kept_positions_gives_back_the_first_pages():
    mgr = CacheManager({0: PagedKVSpec(1, 16, 20)}, page_size=16, n_pages=8, max_len=512)
    mgr.add_request("a")
    mgr.reserve("a", 100)
    mgr.commit("a")
    assert [p >= 0 for p in mgr.requests["a"].pages[0]] == [False] * 5 + [True, True]


# ---- the plain implementation's mechanisms, each against a direct restatement ------------------------------------

def test_plain_sinusoid():
    s = plain.sinusoid(7, 10, torch.float64)
    for p in (0, 3, 6):
        for i in range(5):
            a = p * 10000.0 ** (-2.0 * i / 10)
            assert abs(float(s[p, 2 * i]) - math.sin(a)) < 1e-12 and abs(float(s[p, 2 * i + 1]) - math.cos(a)) < 1e-12
    assert plain.sinusoid(4, 7, torch.float64).shape == (4, 7)          # an odd width ends on a sine


def test_plain_mask():
    see = plain.visible(12, 4, 2)
    assert see[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]
    assert see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert plain.visible(12, 4, 0)[9].nonzero().flatten().tolist() == [6, 7, 8, 9]
    assert plain.visible(5, 100, 0).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()


def test_plain_routing_and_scaled_inputs():
    torch.manual_seed(0)
    D, F, E = 6, 5, 4
    w = {"m.router": torch.randn(E, D, dtype=torch.float64)}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = (torch.randn(F, D, dtype=torch.float64),
                                                                 torch.randn(F, D, dtype=torch.float64),
                                                                 torch.randn(D, F, dtype=torch.float64))
    h = torch.randn(3, D, dtype=torch.float64)
    weight, chosen = plain.route(h, w, "m", 2)
    s = torch.sigmoid(h @ w["m.router"].T)
    for t in range(3):
        order = sorted(range(E), key=lambda e: -float(s[t, e]))[:2]
        assert chosen[t].tolist() == order and torch.allclose(weight[t], s[t, order])
        assert float(weight[t].sum()) != pytest.approx(1.0)           # scores as they are
    out = plain.experts(h, w, "m", {"router": {"top": 2}})
    t, want = 1, torch.zeros(D, dtype=torch.float64)
    for c in range(2):
        e, x = int(chosen[t, c]), weight[t, c] * h[t]
        g, u = w[f"m.e{e}.gate"] @ x, w[f"m.e{e}.up"] @ x
        want += w[f"m.e{e}.down"] @ (g / (1 + torch.exp(-g)) * u)
    assert torch.allclose(out[t], want)
    # the weight on the input is not the weight on the output: the gated unit is not linear
    other = sum(weight[t, c] * plain.gated_unit(h[t:t + 1], w, f"m.e{int(chosen[t, c])}")[0] for c in range(2))
    assert float((other - want).abs().max()) > 1e-3


def test_plain_attention_reads_the_shared_keys_with_its_own_mask():
    config = model(32, 16, [attention(dim=8, heads=2, kv_heads=1, vdim=8, size=3, keep_first=0),
                            attention(dim=8, heads=2, kv_heads=1, vdim=8, size=6, keep_first=1, kv_from=0)])
    d = describe(config)
    w = {k: v.double() for k, v in random_tensors(d, 1).items()}
    toks = list(range(10))
    after, _ = plain.layers(config, w, toks)
    # layer 1 with keys of its own (layer 0's projections applied to ITS input) differs from reading layer 0's keys
    h0 = plain.dynamic_tanh(w["embed"][toks] + plain.sinusoid(10, 16, torch.float64), w, "l0.norm1")
    _, (k0, v0) = plain.attention(h0, w, "l0.mix", config["layers"][0]["mixer"])
    x1 = after[0]
    h1 = plain.dynamic_tanh(x1, w, "l1.norm1")
    y, _ = plain.attention(h1, w, "l1.mix", config["layers"][1]["mixer"], (k0, v0))
    assert torch.allclose(after[1][:, :], x1 + plain.dynamic_tanh(y, w, "l1.norm1b") if config["layers"][1]["mlp"] is None else after[1])
    # causal: a prefix gives the same rows
    assert torch.allclose(plain.forward(config, w, toks)[:6], plain.forward(config, w, toks[:6]))
