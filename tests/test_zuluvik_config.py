"""Zuluvik on the CPU: the configuration reader, the parts it picks, tensor names, the caches of layers that run
another layer's weights, the cache manager's pools with fewer value heads than key heads, the rotation's stretched
frequencies, and the plain implementation's own mechanisms."""
import copy
import math

import pytest
import torch

import plain_zuluvik as plain
from zuluvik_cases import ALL, CONFIG_A, CONFIG_B, CONFIG_ODD, MOE, latent, model, rot, rotary, stretch, two_maps
from mlx_lm_b200.cache import CacheManager
from mlx_lm_b200.config import ConfigError, get_architecture
from mlx_lm_b200.parts import (DifferentialAttention, ExpertsMLP, GatedMLP, LatentAttention, PagedKVSpec, ParallelBlock,
                               RMSNorm, StateSpec, TalkingHeadsAttention, rotation_frequencies)
from mlx_lm_b200.weights.loader import random_tensors


def describe(config):
    arch = get_architecture(config)
    return arch.build(arch.args_class.from_dict(copy.deepcopy(config)))


def test_found_by_its_architecture_key_and_parts_follow_the_layer_list():
    d = describe(CONFIG_A)
    assert d.model_type == "zuluvik"
    assert all(isinstance(b, ParallelBlock) and isinstance(b.norm_1, RMSNorm) for b in d.blocks)
    assert [type(b.mixer) for b in d.blocks] == [LatentAttention, DifferentialAttention, TalkingHeadsAttention, TalkingHeadsAttention]
    assert [type(b.feed_forward) for b in d.blocks] == [ExpertsMLP, ExpertsMLP, type(None), ExpertsMLP]
    assert d.embedding.scale == 4.0 and d.head.tied_to is None and d.position is None
    e = d.blocks[0].feed_forward
    assert (e.n_experts, e.identity, e.n_outputs, e.top, e.groups, e.keep_groups) == (4, 2, 6, 2, 3, 1)
    assert (e.score, e.renormalize, e.scale_input, e.unit, e.limit, e.weight_scale) == ("softmax", True, False, "bounded", 1.0, 1.5)
    assert isinstance(e.shared, GatedMLP) and (e.shared.inner, e.shared.unit, e.shared.limit) == (40, "bounded", 2.0)
    assert d.blocks[1].feed_forward.shared is None and d.blocks[1].feed_forward.groups == 1
    m = d.blocks[1].mixer
    assert (m.n_heads, m.n_kv_heads, m.dim, m.vdim, m.taps, m.diff, m.scale) == (6, 2, 16, 24, 4, 0.3, 0.25)
    r = d.blocks[2].mixer
    assert (r.rot_dims, r.interleaved, r.head_norm, r.has_bias, r.has_out_bias, r.has_talk, r.value_norm) == (24, True, True, True, False, False, False)
    assert d.blocks[3].mixer.rot_scaling is None and r.rot_scaling["factor"] == 8.0
    # the fifth layer runs block 1 again with a cache of its own
    assert [(x.block, x.write) for x in d.runs()] == [(0, True), (1, True), (2, True), (3, True), (1, True)]
    assert len({x.cache_id for x in d.runs()}) == 5


def test_tensor_names_and_shapes():
    d = describe(CONFIG_A)
    specs = {s.name: tuple(s.shape) for s in d.param_specs()}
    D = 64
    assert specs["embed"] == (96, D) and specs["head"] == (96, D) and specs["final.norm"] == (D,)
    assert specs["l0.mix.q"] == (4 * 24, D) and specs["l0.mix.dkv"] == (48, D) and specs["l0.mix.dkv.norm"] == (40,)
    assert specs["l0.mix.uk"] == (64, 40) and specs["l0.mix.uv"] == (96, 40) and specs["l0.mix.o"] == (D, 96)
    assert specs["l0.mlp.router"] == (6, D) and specs["l0.mlp.correction"] == (6,)
    assert specs["l0.mlp.e3.gate"] == specs["l0.mlp.e0.up"] == (24, D) and specs["l0.mlp.e1.down"] == (D, 24)
    assert "l0.mlp.e4.gate" not in specs                      # the two identity experts have no tensors
    assert specs["l0.mlp.shared.gate"] == (40, D) and specs["l0.mlp.shared.down"] == (D, 40)
    assert specs["l1.mix.q"] == (6 * 2 * 16, D) and specs["l1.mix.k"] == (2 * 2 * 16, D) and specs["l1.mix.v"] == (48, D)
    assert specs["l1.mix.q.conv"] == (192, 4) and specs["l1.mix.k.conv"] == (64, 4) and specs["l1.mix.v.conv"] == (48, 4)
    assert specs["l1.mix.lq1"] == specs["l1.mix.lk2"] == (16,) and specs["l1.mix.o"] == (D, 144)
    assert specs["l2.mix.q.b"] == (128,) and specs["l2.mix.k.b"] == (64,) and specs["l2.mix.v.b"] == (32,)
    assert "l2.mix.o.b" not in specs and "l2.mlp.router" not in specs and "l2.norm2" not in specs
    assert not any(k.startswith("l4.") for k in specs)        # the layer that runs layer 1's weights
    only_identity = {s.name for s in describe(CONFIG_B).param_specs()}
    assert "l2.mlp.router" in only_identity and not any(k.startswith("l2.mlp.e") for k in only_identity)
    assert not any(k.startswith(("l1.", "l3.")) for k in only_identity)


def test_caches():
    d = describe(CONFIG_A)
    specs = d.cache_specs()
    own = {x.block: x.cache_id for x in d.runs()[:4]}
    assert specs[own[0]] == PagedKVSpec(1, 48, None, value_dim=0)
    kv = PagedKVSpec(4, 16, None, value_dim=24, value_heads=2)
    assert specs[(own[1], "kv")] == kv and specs[(own[1], "conv")] == StateSpec((3, 192 + 64 + 48))
    second = d.runs()[4].cache_id
    assert specs[(second, "kv")] == kv and specs[(second, "conv")] == StateSpec((3, 304))
    assert specs[own[2]] == PagedKVSpec(2, 32, None, value_dim=16) and specs[own[3]] == PagedKVSpec(2, 16, None, value_dim=32)
    m = CacheManager(specs, page_size=16, n_pages=6, max_requests=2, max_len=64, dtype=torch.float32, device="cpu")
    g = m.kv_groups[m.where((own[1], "kv"))[1]]
    assert g.k.shape == (2, 6, 4, 16, 16) and g.v.shape == (2, 6, 2, 16, 24)        # the two runs of block 1 share a group
    s = m.state_groups[m.where((second, "conv"))[1]]
    assert s.data.shape == (2, 2, 3, 304)
    # a convolution of one tap keeps no state, and none at all asks for none
    one = describe(model(50, 32, [two_maps(conv=1)]))
    assert one.cache_specs() == {0: PagedKVSpec(4, 16, None, value_dim=24, value_heads=2)}
    assert describe(model(50, 32, [two_maps(conv=None)])).blocks[0].mixer.taps == 0


def test_queries_are_ordered_by_key_head_and_map():
    m = DifferentialAttention("x", 32, 6, 2, 4, 8, 0.5, 1e-5, 0.3, taps=2)
    order = m._query_order("cpu").view(-1, 4)[:, 0] // 4           # stored block (head * 2 + map) of every new block
    # new order: key head 0 (map 1 of heads 0, 1, 2; map 2 of heads 0, 1, 2), then key head 1
    assert order.tolist() == [0, 2, 4, 1, 3, 5, 6, 8, 10, 7, 9, 11]


@pytest.mark.parametrize("case", [(16, 10000.0, None), (24, 5000.0, stretch(8.0, 32, 4.0, 1.0)), (64, 50000.0, stretch(16.0, 128)),
                                  (6, 77.0, stretch(3.0, 20, 5.0, 0.7)), (8, 250000.0, stretch(40.0, 4096, 32.0, 1.0))])
def test_stretched_frequencies(case):
    dims, base, scaling = case
    f, mag = rotation_frequencies(dims, base, scaling)
    cos, sin = plain.yarn_table(3, rot(dims, base, scaling))
    assert torch.allclose(cos[1], torch.cos(torch.tensor(f, dtype=torch.float64)) * mag, atol=1e-12)
    assert torch.allclose(sin[2], torch.sin(2 * torch.tensor(f, dtype=torch.float64)) * mag, atol=1e-12)
    if scaling is None:
        assert mag == 1.0 and f == [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    else:
        assert mag == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)
        plainf = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        assert all(a / scaling["factor"] - 1e-15 <= b <= a + 1e-15 for a, b in zip(plainf, f))


def test_configuration_errors():
    bad = lambda edit: (lambda c: (edit(c), c)[1])(copy.deepcopy(CONFIG_A))
    cases = [
        lambda c: c["layers"][0].update(type="wkv"),
        lambda c: c["layers"][1]["mixer"].pop("diff"),
        lambda c: c["layers"][1]["mixer"].update(kv_heads=4),
        lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6),
        lambda c: c["layers"][2]["mixer"]["rot"].update(dims=40),
        lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"),
        lambda c: c["layers"][4].update(weights_of=4),
        lambda c: c["layers"][4].update(weights_of=9),
        lambda c: c["layers"][3].update(weights_of=4),
        lambda c: c["layers"][4]["mixer"].update(scale=0.5),
        lambda c: c["layers"][0]["mlp"].update(kind="dense"),
        lambda c: c["layers"][0]["mlp"]["router"].update(top=7),
        lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4),
        lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4),
        lambda c: c["layers"][3]["mlp"]["router"].update(top=4),       # more than the kept group holds
        lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"),
        lambda c: c.pop("norm"),
        lambda c: c.update(width=0),
    ]
    for edit in cases:
        with pytest.raises(ConfigError):
            describe(bad(edit))
    for name, config in ALL.items():
        describe(config)


def test_random_weights_give_a_working_plain_model():
    for config in (CONFIG_A, CONFIG_B, CONFIG_ODD):
        d = describe(config)
        w = {k: v.float() for k, v in random_tensors(d, 3, torch.bfloat16).items()}
        toks = list(range(20))
        after, logits = plain.layers(config, w, toks)
        assert after.shape == (len(config["layers"]), 20, config["width"]) and torch.isfinite(logits).all()
        # causal: a later token does not move earlier logits
        again_ = plain.forward(config, w, toks[:12] + [7] * 8)
        assert float((again_[:12] - logits[:12]).abs().max()) < 1e-9


def test_plain_route_and_unit():
    h = torch.tensor([[1.0, -2.0, 0.5], [0.1, 0.2, -0.3]], dtype=torch.float64)
    w = {"m.router": torch.tensor([[2.0, 0, 0], [0, 1.0, 0], [0, 0, 3.0], [1.0, 1.0, 1.0], [0.5, 0, 0], [0, 0, 0.1]], dtype=torch.float64),
         "m.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.9, 0.0], dtype=torch.float64)}
    s = torch.softmax(h @ w["m.router"].T, dim=-1)
    weight, chosen = plain.route(h, w, "m", {"top": 2, "scale": 2.0, "experts": 4, "identity": 2})
    assert chosen[:, 0].tolist() == [4, 4]                     # the correction decides the choice ...
    assert torch.allclose(weight.sum(-1), torch.full((2,), 2.0, dtype=torch.float64))
    assert torch.allclose(weight[0, 0] / weight[0, 1], s[0, 4] / s[0, chosen[0, 1]])   # ... and stays out of the weights
    # three groups of two of which one stays: both choices come from the group of expert 4
    _, grouped = plain.route(h, w, "m", {"top": 2, "scale": 1.0, "experts": 4, "identity": 2, "groups": {"count": 3, "keep": 1}})
    assert sorted(grouped[0].tolist()) == [4, 5] and sorted(grouped[1].tolist()) == [4, 5]
    g, u = torch.tensor([[5.0, -1.0]]), torch.tensor([[3.0, -9.0]])
    ww = {"e.gate": torch.eye(2), "e.up": torch.eye(2), "e.down": torch.eye(2)}
    x = torch.tensor([[5.0, -1.0]])
    ww["e.up"] = torch.tensor([[0.6, 0.0], [0.0, 9.0]])
    out = plain.bounded_unit(x, ww, "e", 2.0)
    want0 = 2.0 * torch.sigmoid(torch.tensor(1.702 * 2.0)) * (2.0 + 1.0)          # gate 5 -> 2, up 3 -> 2
    want1 = -1.0 * torch.sigmoid(torch.tensor(-1.702)) * (-2.0 + 1.0)             # gate -1 stays, up -9 -> -2
    assert torch.allclose(out, torch.stack([want0, want1])[None, :])
