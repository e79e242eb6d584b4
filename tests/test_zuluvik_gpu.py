"""Zuluvik through the engine against the plain implementation (tests/plain_zuluvik.py): whole prompts, prefill
against token-by-token decoding, portions down to two tokens, mixed batches with pages and slots that are used
again, each mechanism alone, weights made so that a key lost far back or at a page's border would show, layers that
run another layer's weights with a cache of their own, long decoding, sizes that differ in every place, and greedy
generation through the entry points."""
import copy

import pytest
import torch

import plain_zuluvik as plain
from helpers import Trace, max_live_tokens, mixed_schedule, run_trace
from lelatar_cases import run_engine, tokens, worst
from zuluvik_cases import (ALL, CONFIG_A, CONFIG_B, MOE, ONLY_EXPERTS, ONLY_LATENT, ONLY_ROTARY, ONLY_TWO_MAPS, again, latent,
                           make_dir, model, quiet_embedding, rot, rotary, sharpen, stretch, two_maps)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
# Largest |difference| as a fraction of max(1, largest |logit| of the row).  float32: sums in another order.
# bfloat16: the rounding of every product's inputs, through up to five layers (measured: 0.005 to 0.043).  A key lost
# moves the sharpened models' logits by 0.3 and more.
TOL = {"float32": 1e-5, "bfloat16": 0.055}


def reference(config, weights, requests):
    return {name: plain.forward(config, weights, toks, dtype=torch.float64).float() for name, toks in requests.items()}


def load(path, dtype):
    from mlx_lm_b200.weights import load_model
    return load_model(str(path), dtype=dtype)[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ALL))
def test_whole_prompts(name, dtype, tmp_path):
    """One step per prompt, all logits: also the first tokens of a sequence (lengths 1, 2, 3: shorter than the
    convolutions' taps, so that zeros stand before the start)."""
    config = ALL[name]
    weights = make_dir(tmp_path, config, seed=11, decisive=dtype == "bfloat16")
    reqs = {f"r{n}": tokens(n, config["vocab"], n) for n in (1, 2, 3, 37, 150)}
    tr = Trace()
    for rid, toks in reqs.items():
        tr.whole(rid, toks)
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, reference(config, weights, reqs))
    print(f"whole {name} {dtype}: {w:.3g}")
    assert w < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ALL))
def test_every_cutting_gives_the_same_logits(name, dtype, tmp_path):
    """Prefill then 40 tokens one by one; portions of many sizes (two tokens, one, sizes around 16, 32 and 64 rows,
    more than 128: cuts inside the convolutions' taps and inside pages); mixed batches of unequal requests in a pool
    with three slots and few pages, so that both are used again by later requests."""
    config = ALL[name]
    weights = make_dir(tmp_path, config, seed=5, decisive=dtype == "bfloat16")
    V = config["vocab"]
    reqs = {"a": tokens(70, V, 1), "b": tokens(131, V, 2), "c": tokens(23, V, 3), "d": tokens(300, V, 4), "e": tokens(5, V, 5)}
    tr = Trace()
    for rid, toks in reqs.items():
        tr.bulk_then_single(f"{rid}:tail", toks, tail=40)
    for rid, toks in reqs.items():
        tr.portions(f"{rid}:portions", toks, sizes=(2, 1, 15, 2, 16, 17, 3, 33, 2, 37, 64, 2, 130, 1, 31))
    mixed_schedule(tr, [(f"{rid}:mixed", toks) for rid, toks in reqs.items()], seed=1, max_live=3)
    mixed_schedule(tr, [(f"{rid}:mixed2", toks) for rid, toks in reversed(list(reqs.items()))], seed=2, max_live=3,
                   sizes=(2, 1, 1, 48, 1, 16, 1, 2, 37, 1, 1, 9, 130, 1))
    pool = max_live_tokens(tr, round_to=16)
    got = run_engine(load(tmp_path, dtype), tr, page_size=16, n_pages=pool // 16, max_requests=3, max_len=512)
    assert len(got) == 4 * sum(len(t) for t in reqs.values())
    w = worst(got, reference(config, weights, reqs))
    print(f"cuttings {name} {dtype}: {w:.3g}")
    assert w < TOL[dtype]


SHARP = {
    "two maps": model(64, 48, [two_maps(dim=16, heads=4, kv_heads=2, vdim=16, scale=0.25, diff=0.4, conv=3)]),
    # heads that are normed after the rotation: only the configured scale makes their scores stand out
    "rotary": model(64, 48, [rotary(dim=16, heads=4, kv_heads=2, vdim=16, scale=1.5, rot_=rot(16, 1000.0, stretch(8.0, 64)))]),
    "latent": model(64, 48, [latent(dim=16, heads=4, rot_dim=8, vdim=16, kv_rank=32, scale=0.25, scaling=stretch(8.0, 64))]),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", list(SHARP))
def test_far_keys_and_page_borders(case, dtype, tmp_path):
    """Sharp attention over hundreds of positions: single scores stand out, so a key that is lost (far back, at a
    page's border, at the border of the 64-key blocks the kernels walk, or the sequence's first) moves the logits.
    The plain model that cannot see one position gives other logits; the engine gives the full model's, in portions
    that end at and next to those borders and in decoding."""
    config = SHARP[case]
    weights = make_dir(tmp_path, config, seed=22, edit=lambda w: sharpen(w, 10.0 if case != "rotary" else 1.0))
    V = config["vocab"]
    reqs = {"a": tokens(400, V, 31), "b": tokens(260, V, 32)}
    ref = reference(config, weights, reqs)
    dull = make_dir(tmp_path / "dull", SHARP[case] if case != "rotary" else ALL["rotary"], seed=22)
    dull_cfg = config if case != "rotary" else ALL["rotary"]
    assert float((plain.forward(dull_cfg, dull, reqs["b"]).float() - ref["b"]).abs().max()) > 0.3
    # how much the last positions' logits rest on keys further back than 300, and on the first 64
    short = plain.forward(config, weights, reqs["a"][300:]).float()
    assert float((short[-20:] - ref["a"][-20:]).abs().max()) > 0.3
    tr = Trace()
    tr.portions("a:1", reqs["a"], sizes=(127, 1, 2, 126, 16, 15, 1, 112))
    tr.portions("b:1", reqs["b"], sizes=(129, 127, 2, 2))
    tr.bulk_then_single("b:2", reqs["b"], tail=8)
    tr.bulk_then_single("a:2", reqs["a"], tail=80)
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, ref)
    print(f"far keys {case} {dtype}: {w:.3g}")
    assert w < TOL[dtype]


def test_each_mechanism_matters_and_is_there(tmp_path):
    """The plain model without the second score map, the convolution, the norm of the difference, the rotation's
    stretch, the norm of the heads, the router's correction, the groups, the identity experts, the bounds of the gated
    unit, the shared expert or the embedding's scale gives other logits; the engine gives those of the full one."""
    config = CONFIG_A
    weights = make_dir(tmp_path, config, seed=3, decisive=False, edit=lambda w: sharpen(w, 4.0))
    toks = tokens(60, config["vocab"], 1)
    ref = reference(config, weights, {"a": toks})
    differs = lambda logits: float((logits.float() - ref["a"]).abs().max())
    w64 = {k: v.double() for k, v in weights.items()}
    for name, value in (("l1.mix.lq1", 3.0), ("l1.mix.q.conv", 0.25), ("l1.mix.v.conv", 0.25), ("l0.mlp.correction", 0.0),
                        ("l0.mlp.shared.down", 0.0), ("l2.mix.k.b", 0.0), ("l0.mix.dkv.norm", 1.0)):
        changed = dict(w64)
        changed[name] = torch.full_like(w64[name], value)
        assert differs(plain.forward(config, changed, toks)) > 0.01, name

    def edited(path, value):
        c = copy.deepcopy(config)
        node = c
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        return c
    for path, value in ((("layers", 0, "mixer", "rot", "scaling"), None), (("layers", 2, "mixer", "rot", "scaling"), None),
                        (("layers", 0, "mlp", "router", "groups"), None), (("layers", 0, "mlp", "router", "scale"), 1.0),
                        (("layers", 0, "mlp", "expert", "limit"), 100.0), (("layers", 3, "mlp", "shared", "limit"), 100.0),
                        (("layers", 1, "mixer", "diff"), 0.0), (("embedding", "scale"), 1.0), (("layers", 2, "mixer", "scale"), 0.1),
                        (("norm", "eps"), 0.1)):
        assert differs(plain.forward(edited(path, value), w64, toks)) > 0.01, path
    # the layer that runs layer 1's weights again has a cache of its own: with layer 1's it would see other keys
    once = copy.deepcopy(config)
    once["layers"] = once["layers"][:-1]
    assert differs(plain.forward(once, w64, toks)) > 0.01
    tr = Trace()
    tr.whole("a:w", toks)
    tr.bulk_then_single("a:t", toks, tail=25)
    w = worst(run_engine(load(tmp_path, "float32"), tr), ref)
    assert w < TOL["float32"], w


def test_slots_and_pages_that_are_used_again(tmp_path):
    """One slot and few pages: every request runs in the slot and the pages the one before left behind (the
    convolutions' state starts from zeros again), and gives what it gives alone."""
    config = CONFIG_B
    weights = make_dir(tmp_path, config, seed=2, decisive=False)
    V = config["vocab"]
    a, b = tokens(120, V, 1), tokens(9, V, 2)
    ref = reference(config, weights, {"a": a, "b": b, "c": [3] + a})
    assert float((ref["c"][1:] - ref["a"]).abs().max()) > 0.05
    tr = Trace()
    tr.whole("a:1", a)
    tr.portions("b:1", b, sizes=(2, 1, 3))
    tr.whole("c:1", [3] + a)
    tr.bulk_then_single("a:2", a, tail=30)
    got = run_engine(load(tmp_path, "float32"), tr, max_requests=1, n_pages=16)
    assert worst(got, ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, tmp_path):
    """A short prompt and then 500 tokens one by one beside a second request that comes and goes."""
    config = CONFIG_A
    weights = make_dir(tmp_path, config, seed=8, decisive=dtype == "bfloat16")
    V = config["vocab"]
    reqs = {"a": tokens(510, V, 1), "b": tokens(200, V, 2)}
    ref = reference(config, weights, reqs)
    tr = Trace()
    tr.step([("a", reqs["a"][:10], "all"), ("b", reqs["b"][:3], "all")])
    for t in range(10, 510):
        e = [("a", reqs["a"][t:t + 1], "all")]
        tb = t - 7
        if tb < 200:
            e.append(("b", reqs["b"][tb:tb + 1], "all"))
        tr.step(e, end=(["b"] if tb == 199 else []) + (["a"] if t == 509 else []))
    got = run_engine(load(tmp_path, dtype), tr, n_pages=48, max_requests=2, max_len=640)
    w = worst(got, ref)
    print(f"long decoding {dtype}: {w:.3g}")
    assert w < TOL[dtype]


def test_trace_replay_with_few_slots_and_pages(tmp_path):
    """The command-line replay on this design: mixed steps in a pool that forces pages and slots to be used again."""
    config = CONFIG_B
    weights = make_dir(tmp_path / "m", config, seed=13)
    V = config["vocab"]
    reqs = {f"r{i}": tokens(n, V, 40 + i) for i, n in enumerate((50, 3, 129, 64, 18, 77))}
    ref = reference(config, weights, reqs)
    tr = Trace()
    mixed_schedule(tr, list(reqs.items()), seed=5, max_live=4)
    for dtype in DTYPES:
        got = run_trace(str(tmp_path / "m"), tr, dtype, str(tmp_path / f"out-{dtype}"), extra=("--max-requests", "4"))
        w = worst(got, ref)
        print(f"replay {dtype}: {w:.3g}")
        assert w < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_points(dtype, tmp_path):
    """``generate``, ``stream_generate`` and ``batch_generate`` (scheduler, decode graphs, device sampler) give the
    plain model's greedy tokens."""
    from mlx_lm_b200 import batch_generate, generate, load, stream_generate
    config = CONFIG_A
    weights = make_dir(tmp_path, config, seed=24, edit=quiet_embedding)
    V = config["vocab"]
    prompts = [tokens(9, V, 1), tokens(21, V, 1), tokens(2, V, 2)]

    def greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(plain.forward(config, weights, seq)[-1].argmax()))
        return seq[len(prompt):]

    def agrees(got, ref, prompt):
        for i, (a, b) in enumerate(zip(got, ref)):
            if a != b:
                lg = plain.forward(config, weights, prompt + ref[:i])[-1]
                top = torch.topk(lg, 2).values
                return dtype == "bfloat16" and float(top[0] - top[1]) < 0.05 * float(lg.abs().max())
        return len(got) == len(ref)

    want = [greedy(p, 40) for p in prompts]
    assert all(len(set(w)) >= 4 for w in want), want          # the model does not just repeat itself
    model_, tokenizer = load(str(tmp_path), dtype=dtype)
    for p, w in zip(prompts, want):
        got = [int(t) for t in generate(model_, tokenizer, p, max_tokens=40).split()]
        assert agrees(got, w, p), (got, w)
        streamed = [r.token for r in stream_generate(model_, tokenizer, p, max_tokens=40, prefill_step_size=5)]
        assert agrees(streamed, w, p), (streamed, w)
    out = batch_generate(model_, tokenizer, prompts, max_tokens=40, return_token_ids=True)
    for got, w, p in zip(out.token_ids, want, prompts):
        assert agrees(got, w, p), (got, w)


def test_command_line_and_sampling(tmp_path):
    """`python -m mlx_lm_b200 generate` on a model folder gives the Python entry point's tokens; the random-weights
    mode builds the design from a config.json alone; samplers with filters run on its logits; and what is drawn
    with a temperature does not depend on what else is in the batch."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    from mlx_lm_b200 import generate, load
    from mlx_lm_b200.generate import BatchGenerator
    from mlx_lm_b200.sampling import make_sampler
    config = CONFIG_B
    make_dir(tmp_path / "m", config, seed=31)
    model_, tokenizer = load(str(tmp_path / "m"), dtype="float32")
    want = generate(model_, tokenizer, [5, 17, 3], max_tokens=12)
    run = lambda *a: subprocess.run([sys.executable, "-m", "mlx_lm_b200", "generate", *a], cwd=ROOT, capture_output=True,
                                    text=True, timeout=300)
    r = run("--model", str(tmp_path / "m"), "--prompt", "5 17 3", "-m", "12", "--dtype", "float32", "--verbose", "F")
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == want.split()
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(config))
    r = run("--random-weights", "11", "--config", str(cfg), "--prompt", "5 17 3", "-m", "12", "--temp", "0.7",
            "--top-p", "0.9", "--min-p", "0.01", "--top-k", "20", "--seed", "4", "--verbose", "F")
    assert r.returncode == 0 and len(r.stdout.split()) == 12, r.stderr
    prompts = [tokens(n, config["vocab"], n) for n in (5, 31, 64)]

    def drawn(**kw):
        gen = BatchGenerator(model_, max_tokens=20, sampler=make_sampler(0.8, top_p=0.95), seed=1, **kw)
        uids = gen.insert(prompts)
        out = {u: [] for u in uids}
        while gen.scheduler.has_work():
            for resp in gen.next_generated():
                out[resp.uid].append(resp.token)
        return [out[u] for u in uids]
    together = drawn(completion_batch_size=8, prefill_batch_size=8)
    assert all(len(t) == 20 for t in together)
    assert drawn(completion_batch_size=1, prefill_batch_size=1) == together
    assert drawn(completion_batch_size=2, prefill_batch_size=1, prefill_step_size=7, max_tokens_per_step=9) == together


def drawn_config(seed):
    """A configuration drawn from sizes a small model might have: every layer with a mixer, heads, head sizes, scale
    and rotation of its own, some layers on an earlier layer's weights, feed-forwards of experts or none."""
    import random
    rng = random.Random(seed)
    width = rng.choice([64, 96, 128, 192, 256])
    layers = []
    for i in range(rng.choice([2, 3, 4, 5])):
        own = [j for j, l in enumerate(layers) if "weights_of" not in l]
        if own and rng.random() < 0.3:
            layers.append(again(layers, rng.choice(own)))
            continue
        mlp = None
        if rng.random() < 0.8:
            identity = rng.choice([0, 0, 1, 2, 4])
            experts = rng.choice([2, 4, 6, 8, 12]) if identity else rng.choice([2, 3, 4, 8, 16])
            outputs = experts + identity
            count = rng.choice([c for c in (1, 2, 3, 4) if outputs % c == 0])
            keep = rng.randint(1, count)
            top = rng.choice([t for t in (1, 2, 3, 4) if t <= keep * (outputs // count)])
            mlp = MOE(rng.choice([16, 64, 96, 128]), experts, top, identity=identity, groups=(count, keep) if count > 1 or rng.random() < 0.5 else None,
                      scale=rng.choice([0.5, 1.0, 1.5, 2.5]), limit=rng.choice([0.8, 1.5, 7.0]),
                      shared=(rng.choice([32, 64, 160]), rng.choice([1.0, 2.0])) if rng.random() < 0.6 else None)
        scaling = rng.choice([None, stretch(rng.choice([2.0, 8.0, 40.0]), rng.choice([16, 64, 512]), rng.choice([32.0, 8.0]), rng.choice([1.0, 0.5, 2.0]))])
        kind = rng.choice(["two_maps", "rotary", "latent"])
        heads = rng.choice([2, 4, 6, 8])
        kv = rng.choice([g for g in (1, 2, 3, 4, 8) if heads % g == 0])
        sc = rng.choice([0.09, 0.125, 0.1875, 0.25])
        if kind == "two_maps":
            layers.append(two_maps(dim=rng.choice([16, 32, 64]), heads=heads, kv_heads=kv, vdim=rng.choice([16, 32, 64, 128]), scale=sc,
                                   diff=rng.choice([0.1, 0.3, 0.6]), conv=rng.choice([None, 1, 2, 3, 4, 7]), mlp=mlp))
        elif kind == "rotary":
            dim = rng.choice([16, 32, 64, 128])
            layers.append(rotary(dim=dim, heads=heads, kv_heads=kv, vdim=rng.choice([16, 32, 64, 128]), scale=sc,
                                 rot_=rot(rng.choice([d for d in (0, 8, 16, 32, 64, 128) if d <= dim]), rng.choice([100.0, 10000.0, 500000.0]), scaling),
                                 mlp=mlp))
        else:
            rd = rng.choice([8, 16, 32])
            layers.append(latent(dim=rng.choice([16, 32, 64]), heads=heads, rot_dim=rd, vdim=rng.choice([16, 32, 80]),
                                 kv_rank=rng.choice([24, 64, 96, 160]), scale=sc, base=rng.choice([100.0, 10000.0, 250000.0]),
                                 scaling=scaling, mlp=mlp))
    return model(rng.choice([100, 256, 576, 1000]), width, layers, scale=rng.choice([0.5, 1.0, 8.0]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations(seed, dtype, tmp_path):
    """Whole prompts (one long enough for the experts' many-slot kernels and several attention tiles), prefill and
    decoding, portions and a mixed batch, for configurations nobody picked by hand."""
    config = drawn_config(seed)
    weights = make_dir(tmp_path, config, seed=seed, decisive=dtype == "bfloat16")
    V = config["vocab"]
    reqs = {"a": tokens(600, V, 1), "b": tokens(131, V, 2), "c": tokens(1, V, 3), "d": tokens(77, V, 4)}
    tr = Trace()
    for rid, toks in reqs.items():
        tr.whole(f"{rid}:whole", toks)
    tr.bulk_then_single("b:tail", reqs["b"], tail=40)
    tr.portions("a:portions", reqs["a"], sizes=(2, 129, 1, 64, 3, 200, 17))
    mixed_schedule(tr, [(f"{rid}:mixed", toks) for rid, toks in reqs.items()], seed=seed, max_live=3)
    pool = max_live_tokens(tr, round_to=64)
    got = run_engine(load(tmp_path, dtype), tr, page_size=16, n_pages=pool // 16, max_requests=3, max_len=1024)
    w = worst(got, reference(config, weights, reqs))
    print(f"drawn {seed} {dtype}: {w:.3g}")
    assert w < TOL[dtype]
