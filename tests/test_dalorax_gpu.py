"""Dalorax through the engine against the plain implementation (tests/plain_dalorax.py): whole prompts, prefill
against token-by-token decoding, portions down to two tokens, mixed batches with pages and slots that are used
again, each mechanism alone, weights made so that a key lost or one too many at the edge of a window or of the kept
first positions would show, layers that read another layer's pages, long decoding, sizes that differ in every place,
and greedy generation through the entry points."""
import copy

import pytest
import torch

import plain_dalorax as plain
from dalorax_cases import (CONFIG_A, CONFIG_B, CONFIG_ODD, CONFIG_W, DENSE, MOE, ONLY_ATTENTION, ONLY_EXPERTS, attention, make_dir,
                           model, quiet_embedding, sharpen, with_mask)
from helpers import Trace, max_live_tokens, mixed_schedule, run_trace
from lelatar_cases import run_engine, tokens, worst

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "W": CONFIG_W, "odd": CONFIG_ODD, "attention": ONLY_ATTENTION,
           "experts": ONLY_EXPERTS}
# Largest |difference| as a fraction of max(1, largest |logit| of the row).  float32: sums in another order.
# bfloat16: the rounding of every product's inputs.  A key lost or one too many at an edge moves the sharpened
# models' logits by 0.1 and more.
TOL = {"float32": 5e-6, "bfloat16": 0.02}


def reference(config, weights, requests):
    return {name: plain.forward(config, weights, toks, dtype=torch.float64).float() for name, toks in requests.items()}


def load(path, dtype):
    from mlx_lm_b200.weights import load_model
    return load_model(str(path), dtype=dtype)[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts(name, dtype, tmp_path):
    """One step per prompt, all logits: also the first tokens of a sequence (lengths 1, 2, 3: the first window is
    not full, kept positions and window overlap)."""
    config = CONFIGS[name]
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
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_gives_the_same_logits(name, dtype, tmp_path):
    """Prefill then 40 tokens one by one; portions of many sizes (two tokens, one, sizes around 16, 32 and 64 rows,
    more than 128); mixed batches of unequal requests in a pool with three slots and few pages, so that both are used
    again by later requests."""
    config = CONFIGS[name]
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


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["window", "kept first positions", "a reader's wider window"])
def test_keys_at_the_edges_of_windows_and_of_the_kept_positions(case, dtype, tmp_path):
    """Sharp attention: single scores stand out.  The plain model with a window, or a number of kept positions, one
    longer or shorter gives other logits (so a key lost or one too many at the edge shows), and the engine gives the
    plain model's: in prompts cut at, just before and just after the edges, and in tokens decoded one by one across
    them."""
    if case == "window":
        config, layer, key, size = copy.deepcopy(ONLY_ATTENTION), 0, "size", 30
    elif case == "kept first positions":
        config, layer, key, size = with_mask(ONLY_ATTENTION, 0, size=11, keep_first=19), 0, "keep_first", 19
    else:
        # layer 1 reads layer 0's pages through a window three times as wide, and keeps positions layer 0 does not
        config = model(64, 48, [attention(dim=16, heads=4, kv_heads=2, vdim=16, scale=0.25, softcap=40.0, size=12, keep_first=0),
                                attention(dim=16, heads=4, kv_heads=2, vdim=16, scale=0.25, softcap=40.0, size=36, keep_first=6,
                                          kv_from=0)])
        layer, key, size = 1, "size", 36
    weights = make_dir(tmp_path, config, seed=21, edit=lambda w: sharpen(w, 12.0))
    V = config["vocab"]
    reqs = {"a": tokens(135, V, 31), "b": tokens(90, V, 32)}
    ref = reference(config, weights, reqs)
    for other in (size - 1, size + 1):
        moved = plain.forward(with_mask(config, layer, **{key: other}), weights, reqs["a"]).float()
        assert float((moved - ref["a"]).abs().max()) > 0.3, other
    tr = Trace()
    tr.whole("a:w", reqs["a"])
    tr.portions("a:1", reqs["a"], sizes=(size - 1, 1, 1, size - 2, 2, 2, size, 3))
    tr.portions("b:1", reqs["b"], sizes=(size, size - 1, 2, 2))
    tr.bulk_then_single("a:2", reqs["a"], tail=135 - size + 3)           # decodes across every edge after the first
    tr.bulk_then_single("b:2", reqs["b"], tail=12)
    tr.bulk_then_single("b:3", reqs["b"], tail=88)                       # the kept positions themselves are decoded
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, ref)
    print(f"edges: {case} {dtype}: {w:.3g}")
    assert w < 2 * TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_and_page_borders(dtype, tmp_path):
    """Windows of hundreds of positions with sharp attention: keys far back, across many pages and across the 64-key
    blocks the kernel walks, in portions that end at and next to those borders and in decoding; and kept first
    positions hundreds of positions behind a narrow window."""
    config = copy.deepcopy(CONFIG_A)
    config["layers"][0]["mixer"]["mask"]["size"] = 333
    config["layers"][1]["mixer"]["mask"]["size"] = 290
    config["layers"][2]["mixer"]["mask"].update(size=17, keep_first=66)
    config["layers"][3]["mixer"]["mask"]["size"] = 256
    weights = make_dir(tmp_path, config, seed=22, edit=lambda w: sharpen(w, 8.0))
    V = config["vocab"]
    reqs = {"a": tokens(400, V, 31), "b": tokens(260, V, 32)}
    ref = reference(config, weights, reqs)
    dull = make_dir(tmp_path / "dull", config, seed=22)
    assert float((plain.forward(config, dull, reqs["b"]).float() - ref["b"]).abs().max()) > 0.5
    for layer, mask in ((2, {"keep_first": 65}), (2, {"keep_first": 67}), (0, {"size": 332}), (3, {"size": 257})):
        moved = plain.forward(with_mask(config, layer, **mask), weights, reqs["a"]).float()
        assert float((moved - ref["a"]).abs().max()) > 0.1, (layer, mask)
    tr = Trace()
    tr.portions("a:1", reqs["a"], sizes=(127, 1, 2, 126, 16, 15, 1, 112))
    tr.portions("b:1", reqs["b"], sizes=(129, 127, 2, 2))
    tr.bulk_then_single("b:2", reqs["b"], tail=8)
    tr.bulk_then_single("a:2", reqs["a"], tail=80)
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, ref)
    print(f"far keys {dtype}: {w:.3g}")
    assert w < 2 * TOL[dtype]


def test_each_mechanism_matters_and_is_there(tmp_path):
    """The plain model without the gate, the soft cap, the norm after a sublayer, the sinusoid, the shared pages, or
    with the routing weight on the experts' output instead of their input gives other logits; the engine gives those
    of the full one."""
    config = CONFIG_A
    weights = make_dir(tmp_path, config, seed=3, edit=lambda w: sharpen(w, 6.0))
    toks = tokens(60, config["vocab"], 1)
    ref = reference(config, weights, {"a": toks})
    differs = lambda logits: float((logits.float() - ref["a"]).abs().max())
    w64 = {k: v.double() for k, v in weights.items()}
    for name, value in (("l0.mix.g", 0.0), ("l2.norm1b.alpha", 1e-3), ("l1.norm2b.b", 0.0), ("l1.mlp.router", 0.0)):
        changed = dict(w64)
        changed[name] = torch.full_like(w64[name], value)
        assert differs(plain.forward(config, changed, toks)) > 0.02, name
    uncapped = copy.deepcopy(config)
    for layer in uncapped["layers"]:
        layer["mixer"]["softcap"] = 0.0
    assert differs(plain.forward(uncapped, w64, toks)) > 0.02
    own = copy.deepcopy(config)                       # layer 2 with layer 0's projections on its own input
    del own["layers"][2]["mixer"]["kv_from"]
    own_w = dict(w64, **{"l2.mix.k": w64["l0.mix.k"], "l2.mix.v": w64["l0.mix.v"]})
    assert differs(plain.forward(own, own_w, toks)) > 0.02
    shifted = plain.forward(config, w64, [0] + toks)[1:]     # every position one further on: the sinusoid moves
    assert differs(shifted) > 0.02
    tr = Trace()
    tr.whole("a:w", toks)
    tr.bulk_then_single("a:t", toks, tail=25)
    w = worst(run_engine(load(tmp_path, "float32"), tr), ref)
    assert w < TOL["float32"], w


def test_the_position_enters_only_at_the_embedding(tmp_path):
    """Two requests with the same tokens at other positions (one has a token in front) differ; the same tokens at
    the same positions give the same logits whatever ran in the slot and the pages before."""
    config = ONLY_EXPERTS
    weights = make_dir(tmp_path, config, seed=2)
    V = config["vocab"]
    a, b = tokens(120, V, 1), tokens(9, V, 2)
    ref = reference(config, weights, {"a": a, "b": b, "c": [3] + a})
    assert float((ref["c"][1:] - ref["a"]).abs().max()) > 0.05
    tr = Trace()
    tr.whole("a:1", a)
    tr.portions("b:1", b, sizes=(2, 1, 3))
    tr.whole("c:1", [3] + a)
    tr.whole("a:2", a)
    got = run_engine(load(tmp_path, "float32"), tr, max_requests=1, n_pages=16)
    assert worst(got, ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, tmp_path):
    """A short prompt and then 500 tokens one by one beside a second request: windows pass over decoded tokens many
    times, pages behind the windows are given back and taken again while those of the kept positions stay."""
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
    got = run_engine(load(tmp_path, dtype), tr, n_pages=24, max_requests=2, max_len=640)
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

    want = [greedy(p, 60) for p in prompts]
    assert all(len(set(w)) >= 4 for w in want), want          # the model does not just repeat itself
    model_, tokenizer = load(str(tmp_path), dtype=dtype)
    for p, w in zip(prompts, want):
        got = [int(t) for t in generate(model_, tokenizer, p, max_tokens=60).split()]
        assert agrees(got, w, p), (got, w)
        streamed = [r.token for r in stream_generate(model_, tokenizer, p, max_tokens=60, prefill_step_size=5)]
        assert agrees(streamed, w, p), (streamed, w)
    out = batch_generate(model_, tokenizer, prompts, max_tokens=60, return_token_ids=True)
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
    """A configuration drawn from sizes a small model might have: every layer with heads, head sizes, mask, scale and
    cap of its own, some layers on an earlier layer's pages, feed-forwards dense, of experts, or none."""
    import random
    rng = random.Random(seed)
    width = rng.choice([64, 96, 128, 192, 256])
    layers = []
    for i in range(rng.choice([2, 3, 4, 5])):
        owners = [j for j, l in enumerate(layers) if "kv_from" not in l["mixer"]]
        mask = dict(size=rng.choice([3, 17, 40, 64, 100, 300]), keep_first=rng.choice([0, 1, 4, 16, 70]))
        kw = dict(scale=rng.choice([0.09, 0.125, 0.1875, 0.25]), softcap=rng.choice([5.0, 20.0, 30.0, 50.0]), **mask)
        mlp = rng.choice([None, "dense", "moe", "moe"])
        if mlp == "dense":
            mlp = DENSE(rng.choice([64, 96, 256, 320]))
        elif mlp == "moe":
            experts = rng.choice([2, 4, 8, 12, 16])
            mlp = MOE(rng.choice([16, 64, 96, 128]), experts, rng.choice([t for t in (1, 2, 4) if t <= experts]))
        if owners and rng.random() < 0.4:
            j = rng.choice(owners)
            m = layers[j]["mixer"]
            layers.append(attention(dim=m["dim"], heads=m["heads"], kv_heads=m["kv_heads"], vdim=m["vdim"], kv_from=j, mlp=mlp, **kw))
        else:
            heads = rng.choice([2, 4, 6, 8])
            layers.append(attention(dim=rng.choice([16, 32, 64, 64, 128]), heads=heads,
                                    kv_heads=rng.choice([g for g in (1, 2, 3, 4, 8) if heads % g == 0]),
                                    vdim=rng.choice([16, 32, 64, 64, 128]), mlp=mlp, **kw))
    return model(rng.choice([100, 256, 576, 1000]), width, layers, logit_scale=rng.choice([0.5, 1.0, 2.0]))


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
