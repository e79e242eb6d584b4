"""Small Zuluvik configurations for the tests and model folders with seeded random weights."""
import copy
import math
import os

import torch
from safetensors.torch import load_file, save_file


def stretch(factor, original, fast=32.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def rot(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = scaling
    return r


def two_maps(dim=16, heads=4, kv_heads=2, vdim=24, scale=0.25, diff=0.3, conv=4, mlp=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale, "diff": diff}
    if conv is not None:
        mixer["conv"] = conv
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def rotary(dim=32, heads=4, kv_heads=2, vdim=16, scale=0.2, rot_=None, mlp=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale}
    if rot_ is not None:
        mixer["rot"] = rot_
    return {"type": "attention_2", "mixer": mixer, "mlp": mlp}


def latent(dim=16, heads=4, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, base=10000.0, scaling=None, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": rot(rot_dim, base, scaling)}}


def MOE(ff, experts, top, identity=0, groups=None, scale=1.0, limit=1.5, shared=None):
    router = {"experts": experts, "top": top, "identity": identity, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def again(layers, j):
    """Layer ``j`` once more: the same entry, ``weights_of: j``."""
    return dict(copy.deepcopy(layers[j]), weights_of=j)


def model(vocab, width, layers, scale=1.0, eps=1e-5):
    return {"architecture": "Zuluvik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": layers}


# Different from one another in every size; what is equal or 1 in one is not in the others.
# A: every kind of mixer, three query heads a key head, a rotation of part of the head with a stretch that is active
# among the pairs, two identity experts, three groups of which one stays, a layer without a feed-forward, and layer 1
# once more at the end
_A = [latent(dim=16, heads=4, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, scaling=stretch(4.0, 64, fast=8.0, slow=0.5),
             mlp=MOE(24, 4, 2, identity=2, groups=(3, 1), scale=1.5, limit=1.0, shared=(40, 2.0))),
      two_maps(dim=16, heads=6, kv_heads=2, vdim=24, scale=0.25, diff=0.3, conv=4, mlp=MOE(32, 5, 3, identity=1, scale=0.8)),
      rotary(dim=32, heads=4, kv_heads=2, vdim=16, scale=0.2, rot_=rot(24, 5000.0, stretch(8.0, 32, fast=4.0, slow=1.0))),
      rotary(dim=16, heads=2, kv_heads=2, vdim=32, scale=0.3, rot_=rot(16, 100.0),
             mlp=MOE(16, 6, 1, groups=(2, 1), limit=0.7, shared=(24, 0.9)))]
CONFIG_A = model(96, 64, _A + [again(_A, 1)], scale=4.0)
# B: one key head for all, heads of 48 and 40, a convolution of two taps, every group kept, all experts chosen,
# identity experts only (no expert with tensors) in one layer, no shared expert, a layer that runs three times
_B = [two_maps(dim=48, heads=3, kv_heads=1, vdim=40, scale=0.15, diff=0.55, conv=2, mlp=MOE(128, 3, 3, groups=(3, 3), scale=2.0, limit=3.0)),
      latent(dim=24, heads=6, rot_dim=16, vdim=8, kv_rank=72, scale=0.18, base=300.0,
             mlp=MOE(8, 0, 2, identity=4, groups=(2, 2), scale=0.5, shared=(64, 1.2)))]
CONFIG_B = model(200, 96, [_B[0], again(_B, 0), _B[1], again(_B, 0)], scale=0.5, eps=1e-6)
# W: sizes of a larger model's heads: eight heads of 64 over two key heads, latent rows of 128 + 32, sixteen router
# outputs and sixteen experts
CONFIG_W = model(128, 128, [rotary(dim=64, heads=8, kv_heads=2, vdim=64, scale=0.125, rot_=rot(64, 50000.0, stretch(16.0, 128)),
                                   mlp=MOE(96, 10, 4, identity=6, groups=(4, 2), scale=2.5, limit=2.5, shared=(192, 2.0))),
                            two_maps(dim=64, heads=8, kv_heads=4, vdim=64, scale=0.125, diff=0.2, conv=3, mlp=MOE(64, 16, 2)),
                            latent(dim=64, heads=8, rot_dim=32, vdim=64, kv_rank=128, scale=0.1, scaling=stretch(2.0, 256, 16.0, 2.0))],
                 scale=8.0)
# nothing is a multiple of 8: every 16-byte path steps aside (products, pages, the tensor-core attention and experts)
CONFIG_ODD = model(77, 50, [two_maps(dim=6, heads=3, kv_heads=3, vdim=10, scale=0.4, diff=0.1, conv=5, mlp=MOE(14, 5, 2, identity=1, groups=(2, 1))),
                            rotary(dim=12, heads=3, kv_heads=1, vdim=10, scale=0.3, rot_=rot(6, 77.0, stretch(3.0, 20, 5.0, 0.7)),
                                   mlp=MOE(30, 3, 2, shared=(22, 1.1))),
                            latent(dim=10, heads=5, rot_dim=6, vdim=14, kv_rank=21, scale=0.35, base=50.0)],
                   scale=3.0)
ONLY_TWO_MAPS = model(64, 48, [two_maps(dim=16, heads=4, kv_heads=2, vdim=16, scale=0.25, diff=0.4, conv=3)])
ONLY_ROTARY = model(64, 48, [rotary(dim=16, heads=4, kv_heads=2, vdim=16, scale=0.25, rot_=rot(16, 1000.0, stretch(8.0, 64)))])
ONLY_LATENT = model(64, 48, [latent(dim=16, heads=4, rot_dim=8, vdim=16, kv_rank=32, scale=0.25, scaling=stretch(8.0, 64))])
ONLY_EXPERTS = model(64, 48, [rotary(dim=16, heads=2, kv_heads=1, vdim=16, scale=0.25, rot_=rot(8),
                                     mlp=MOE(32, 6, 2, identity=2, groups=(4, 3), scale=1.5, shared=(40, 2.0)))])

ALL = {"A": CONFIG_A, "B": CONFIG_B, "W": CONFIG_W, "odd": CONFIG_ODD, "two maps": ONLY_TWO_MAPS, "rotary": ONLY_ROTARY,
       "latent": ONLY_LATENT, "experts": ONLY_EXPERTS}


CODE_COLUMNS = 3
CODE_SIZE = 4000.0
CODE_WEIGHT = 0.3        # the norms' weight in the code columns


def route_margins(z, correction, router):
    """For router logits ``z [n, outputs]``: the smallest gap, over the rows, between the last choice score that is
    taken and the first that is not (among groups, then among the outputs of the kept groups), as a fraction of the
    larger of the two scores (a rounding of the logits moves a score by a fraction of itself)."""
    s = torch.softmax(z, dim=-1) + correction
    gap = math.inf
    rel = lambda a, b: float(((a - b) / torch.maximum(a.abs(), b.abs()).clamp_min(1e-3)).min())
    groups = router.get("groups")
    if groups and groups["keep"] < groups["count"]:
        per = s.shape[1] // groups["count"]
        best = s.view(-1, groups["count"], per).max(dim=-1).values.sort(dim=-1, descending=True).values
        gap = min(gap, rel(best[:, groups["keep"] - 1], best[:, groups["keep"]]))
        kept = torch.topk(s.view(-1, groups["count"], per).max(dim=-1).values, groups["keep"], dim=-1).indices
        allowed = torch.zeros(s.shape[0], groups["count"], dtype=torch.bool).scatter_(1, kept, True)
        s = s.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    top = router["top"]
    order = s.sort(dim=-1, descending=True).values
    if top < s.shape[1]:
        ok = torch.isfinite(order[:, top])
        if ok.any():
            gap = min(gap, rel(order[ok, top - 1], order[ok, top]))
    return gap


def decisive_routers(w, config, seed, gap=0.08):
    """Routers that never face a close call, so that bfloat16 rounding cannot send a token to another expert than
    float64 does.  The first few columns of the embedding hold +-CODE_SIZE (after the embedding's scale) and no layer
    writes to these columns of the stream, so the normed input of every feed-forward has, in these columns, one of
    2^CODE_COLUMNS sign patterns times a factor that depends a little on the rest of the row (the code columns are
    so large that they make up nearly all of a row's mean square; the norms' weights in the other columns are raised by
    as much, so that the layers' inputs there stay of size 1).  The routers read only
    these columns and are drawn again until, for every pattern and every factor in the range, the last group and the
    last expert taken are ``gap`` above the next.  The model's last norm is zero in these columns."""
    g = torch.Generator().manual_seed(1000 + seed)
    n, D = CODE_COLUMNS, config["width"]
    rounded = lambda t: t.to(torch.bfloat16).float()
    w["embed"][:, :n] = CODE_SIZE / config["embedding"]["scale"] * (torch.randint(0, 2, (config["vocab"], n), generator=g) * 2 - 1).float()
    w["final.norm"][:n] = 0.0
    boost = CODE_SIZE * math.sqrt(n / D)         # about the root mean square of a row: the other columns stay of size 1
    w["final.norm"][n:] *= boost
    signs = torch.tensor([[1.0 if (p >> c) & 1 else -1.0 for c in range(n)] for p in range(2 ** n)])
    for i, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        for k in list(w):
            if k.startswith(f"l{i}.") and (k.endswith(".mix.o") or k.endswith(".down")):
                w[k][:n] = 0.0                       # the rows that make the stream's code columns
        w[f"l{i}.norm1"][:n] = CODE_WEIGHT
        w[f"l{i}.norm1"][n:] *= boost
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        router = mlp["router"]
        outputs = router["experts"] + router.get("identity", 0)
        corr = rounded(w[f"l{i}.mlp.correction"])
        # the code columns of the normed row: sign * CODE_SIZE / rms * weight, rms between that of a row with
        # nothing else in it and that of a row whose other columns are as large as the code columns
        full = math.sqrt(D / n)
        for attempt in range(20000):
            r = rounded((0.5, 1.0, 2.0)[attempt % 3] * torch.randn(outputs, n, generator=g))
            ok = True
            for factor in (1.0, 0.995, 0.985, 0.97, 0.94):
                h = rounded(signs * full * factor * CODE_WEIGHT)
                if route_margins(h @ r.T, corr, router) <= gap:
                    ok = False
                    break
            if ok:
                break
        else:
            raise RuntimeError(f"no decisive router for layer {i}")
        w[f"l{i}.mlp.router"] = torch.zeros_like(w[f"l{i}.mlp.router"])
        w[f"l{i}.mlp.router"][:, :n] = r


def make_dir(path, config, seed, edit=None, decisive=True):
    """A model folder with random weights; ``edit(tensors)`` may change them (float32 in, rounded to bfloat16 again).
    ``decisive``: routers without close calls (``decisive_routers``); without it they are as random as the rest,
    which suits float32 runs only."""
    from mlx_lm_b200.weights import write_random_model

    write_random_model(str(path), copy.deepcopy(config), seed)
    file = os.path.join(str(path), "model.safetensors")
    w = {k: v.float() for k, v in load_file(file).items()}
    if decisive:
        decisive_routers(w, config, seed)
    if edit is not None:
        edit(w)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, file)
    return load_file(file)


def sharpen(w, factor):
    """Queries scaled up so that single scores stand out: a key that is lost, or one too many, moves the logits."""
    for k in w:
        if k.endswith(".mix.q") or k.endswith(".mix.q.b"):
            w[k] *= factor


def quiet_embedding(w, factor=0.04):
    """The embedding scaled down (but for the routers' code columns), so that the layers and not the last token's own
    row decide the next token: greedy generation then wanders instead of repeating itself."""
    w["embed"][:, CODE_COLUMNS:] *= factor
