"""Small Dalorax configurations for the tests and model folders with seeded random weights."""
import copy
import os

import torch
from safetensors.torch import load_file, save_file


def attention(dim=32, heads=4, kv_heads=2, vdim=16, scale=0.2, softcap=8.0, size=24, keep_first=3, kv_from=None, mlp=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale, "softcap": softcap,
             "mask": {"size": size, "keep_first": keep_first}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mlp": mlp, "mixer": mixer}


DENSE = lambda ff: {"ff": ff, "kind": "dense"}
MOE = lambda ff, experts, top: {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, layers, logit_scale=1.0, eps=1e-5):
    return {"architecture": "Dalorax", "vocab": vocab, "width": width, "logit_scale": logit_scale, "norm": {"eps": eps},
            "layers": layers}


# Different from one another in every size; what is equal or 1 in one is not in the others.
# A: two experts a token; a layer without a feed-forward that reads layer 0's pages through a WIDER window and with
# more kept positions than layer 0 itself; a last layer with keys of its own again
CONFIG_A = model(96, 64, [attention(mlp=DENSE(80)),
                          attention(dim=16, heads=2, kv_heads=1, vdim=32, size=40, keep_first=0, scale=0.3, mlp=MOE(24, 6, 2)),
                          attention(kv_from=0, size=50, keep_first=5, scale=0.15, softcap=3.0),
                          attention(dim=32, heads=4, kv_heads=4, vdim=16, size=9, keep_first=1, mlp=MOE(40, 3, 1))],
                 logit_scale=1.5)
# B: every head with keys of its own, heads of 48 and 40, a window of two positions, kept positions beyond a block of
# 64 keys and beyond the window, three of five experts, a feed-forward wider than the model, logits scaled down
CONFIG_B = model(200, 96, [attention(dim=48, heads=3, kv_heads=3, vdim=40, size=2, keep_first=70, scale=0.15, softcap=20.0,
                                     mlp=MOE(128, 5, 3)),
                           attention(dim=24, heads=6, kv_heads=2, vdim=8, size=100, keep_first=7, scale=0.25, mlp=DENSE(256)),
                           attention(dim=24, heads=6, kv_heads=2, vdim=8, size=33, keep_first=90, kv_from=1, scale=0.2,
                                     softcap=2.0, mlp=MOE(16, 9, 9))],
                 logit_scale=0.5, eps=1e-6)
# W: sizes of a larger model's heads: eight heads of 64 over two key heads, windows over several blocks, sixteen experts
CONFIG_W = model(128, 128, [attention(dim=64, heads=8, kv_heads=2, vdim=64, size=130, keep_first=4, scale=0.125, softcap=30.0,
                                      mlp=MOE(64, 16, 2)),
                            attention(dim=64, heads=8, kv_heads=2, vdim=64, size=64, keep_first=64, kv_from=0, scale=0.1,
                                      mlp=DENSE(192)),
                            attention(dim=128, heads=2, kv_heads=1, vdim=64, size=300, keep_first=1, scale=0.09, softcap=50.0)])
# nothing is a multiple of 8: every 16-byte path steps aside (products, pages, the tensor-core attention and experts)
CONFIG_ODD = model(77, 50, [attention(dim=12, heads=3, kv_heads=1, vdim=10, size=9, keep_first=2, scale=0.3, mlp=MOE(14, 5, 2)),
                            attention(dim=12, heads=3, kv_heads=1, vdim=10, size=11, keep_first=3, kv_from=0, scale=0.3,
                                      mlp=DENSE(30)),
                            attention(dim=6, heads=5, kv_heads=5, vdim=14, size=21, keep_first=0, scale=0.4, softcap=1.5)],
                   logit_scale=3.0)
ONLY_ATTENTION = model(64, 48, [attention(dim=16, heads=4, kv_heads=2, vdim=16, scale=0.25, softcap=40.0, size=30, keep_first=4)])
ONLY_EXPERTS = model(64, 48, [attention(dim=16, heads=2, kv_heads=1, vdim=16, size=1000, keep_first=0, mlp=MOE(32, 8, 2))])

ALL = {"A": CONFIG_A, "B": CONFIG_B, "W": CONFIG_W, "odd": CONFIG_ODD, "attention": ONLY_ATTENTION, "experts": ONLY_EXPERTS}


CODE_COLUMNS = 5


def decisive_routers(w, config, seed, gap=0.1):
    """Routers that never face a close call, so that bfloat16 rounding cannot send a token to another expert than
    float64 does.  The first few columns of the embedding hold +-30: the norms' tanh saturates there whatever the
    layers add, so the feed-forward's input has one of 2^CODE_COLUMNS fixed patterns in these columns.  The routers
    read only these columns and are drawn again until, for every pattern, the last chosen expert's logit is ``gap``
    above the next one's.  The model's last norm is zero in these columns, so they do not reach the logits."""
    g = torch.Generator().manual_seed(1000 + seed)
    n = CODE_COLUMNS
    w["embed"][:, :n] = 30.0 * (torch.randint(0, 2, (config["vocab"], n), generator=g) * 2 - 1).float()
    w["final.norm"][:n] = 0.0
    w["final.norm.b"][:n] = 0.0
    signs = torch.tensor([[1.0 if (p >> c) & 1 else -1.0 for c in range(n)] for p in range(2 ** n)])
    rounded = lambda t: t.to(torch.bfloat16).float()
    for i, layer in enumerate(config["layers"]):
        mlp = layer.get("mlp")
        if mlp is None or mlp["kind"] != "moe":
            continue
        E, top = mlp["router"]["experts"], mlp["router"]["top"]
        h = rounded(signs * torch.sign(w[f"l{i}.norm2.alpha"]) * rounded(w[f"l{i}.norm2"][:n]) + rounded(w[f"l{i}.norm2.b"][:n]))
        for _ in range(100000):
            r = rounded(2.0 * torch.randn(E, n, generator=g))
            z = (h @ r.T).sort(dim=-1, descending=True).values
            if top == E or float((z[:, top - 1] - z[:, top]).min()) > gap:
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
        if k.endswith(".mix.q"):
            w[k] *= factor


def quiet_embedding(w, factor=0.04):
    """The embedding scaled down (but for the routers' code columns), so that the layers and not the last token's own
    row decide the next token: greedy generation then wanders instead of repeating itself."""
    w["embed"][:, CODE_COLUMNS:] *= factor


def with_mask(config, layer, **mask):
    c = copy.deepcopy(config)
    c["layers"][layer]["mixer"]["mask"].update(mask)
    return c
