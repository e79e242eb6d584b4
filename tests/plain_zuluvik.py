"""A plain, slow Zuluvik: whole sequences through straightforward torch code, one function per mechanism, written
from the design's equations and sharing nothing with the package.  ``weights``: tensor name -> tensor as stored."""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def yarn_table(n, rot, dtype=torch.float64):
    """(cos, sin) of every position's angles, ``[n, dims / 2]``, with the frequencies stretched as the scaling asks
    and both tables times its magnitude factor."""
    dims, base = rot["dims"], float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        def where(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        i = torch.arange(dims // 2, dtype=torch.float64)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    a = torch.arange(n, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(a) * mag).to(dtype), (torch.sin(a) * mag).to(dtype)


def turn(x, cos, sin, dims):
    """``x [T, heads, d]``: the first ``dims`` of every head turned, pairs (2i, 2i+1)."""
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_softmax_values(q, k, v, scale):
    """One head: ``q [T, d]``, ``k [T, d]``, ``v [T, e]``."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
    return torch.softmax(s, dim=-1) @ v


def short_convolution(u, taps_weight):
    """``u [T, C]``, ``taps_weight [C, taps]``: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u])
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_weight[:, j].to(u.dtype)[None, :]
    return y


def differential_attention(h, w, name, m, eps):
    T, dt = h.shape[0], h.dtype
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w[f"{name}.{n}"].to(dt).T for n in "qkv")
    if m.get("conv"):
        q, k, v = (short_convolution(t, w[f"{name}.{n}.conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, 2, d), k.view(T, G, 2, d), v.view(T, G, e)
    f = lambda n: w[f"{name}.{n}"].to(dt)
    lam = torch.exp((f("lq1") * f("lk1")).sum()) - torch.exp((f("lq2") * f("lk2")).sum()) + m["diff"]
    heads = []
    for a in range(H):
        c = a // (H // G)
        first = causal_softmax_values(q[:, a, 0], k[:, c, 0], v[:, c], m["scale"])
        second = causal_softmax_values(q[:, a, 1], k[:, c, 1], v[:, c], m["scale"])
        heads.append(rms(first - lam * second, eps) * (1.0 - m["diff"]))
    return torch.cat(heads, dim=-1) @ w[name + ".o"].to(dt).T


def rotary_attention(h, w, name, m, eps):
    T, dt = h.shape[0], h.dtype
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w[f"{name}.{n}"].to(dt).T + w[f"{name}.{n}.b"].to(dt) for n in "qkv")
    cos, sin = yarn_table(T, m["rot"], dt)
    q = rms(turn(q.view(T, H, d), cos, sin, m["rot"]["dims"]), eps)
    k = rms(turn(k.view(T, G, d), cos, sin, m["rot"]["dims"]), eps)
    v = v.view(T, G, e)
    heads = [causal_softmax_values(q[:, a], k[:, a // (H // G)], v[:, a // (H // G)], m["scale"]) for a in range(H)]
    return torch.cat(heads, dim=-1) @ w[name + ".o"].to(dt).T


def latent_attention(h, w, name, m, eps):
    T, dt = h.shape[0], h.dtype
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[name + ".q"].to(dt).T).view(T, H, d + r)
    down = h @ w[name + ".dkv"].to(dt).T
    c = rms(down[:, :R], eps) * w[name + ".dkv.norm"].to(dt)
    cos, sin = yarn_table(T, m["rot"], dt)
    k_turned = turn(down[:, None, R:], cos, sin, r)[:, 0]
    q_turned = turn(q[:, :, d:], cos, sin, r)
    keys = (c @ w[name + ".uk"].to(dt).T).view(T, H, d)
    values = (c @ w[name + ".uv"].to(dt).T).view(T, H, e)
    heads = []
    for a in range(H):
        qa = torch.cat([q[:, a, :d], q_turned[:, a]], dim=-1)
        ka = torch.cat([keys[:, a], k_turned], dim=-1)
        heads.append(causal_softmax_values(qa, ka, values[:, a], m["scale"]))
    return torch.cat(heads, dim=-1) @ w[name + ".o"].to(dt).T


def bounded_unit(h, w, name, limit):
    dt = h.dtype
    g = (h @ w[name + ".gate"].to(dt).T).clamp(max=limit)
    u = (h @ w[name + ".up"].to(dt).T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[name + ".down"].to(dt).T


def route(h, w, name, router):
    """(weights [T, top], experts [T, top]); numbers from ``experts`` on stand for identity experts."""
    s = torch.softmax(h @ w[name + ".router"].to(h.dtype).T, dim=-1)
    choice = s + w[name + ".correction"].to(h.dtype)
    groups = router.get("groups")
    if groups:
        per = choice.shape[1] // groups["count"]
        best = choice.view(-1, groups["count"], per).max(dim=-1).values
        kept = torch.topk(best, groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = torch.topk(choice, router["top"], dim=-1).indices
    weight = torch.gather(s, 1, chosen)
    return weight / (weight.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"], chosen


def experts(h, w, name, mlp):
    router = mlp["router"]
    weight, chosen = route(h, w, name, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(chosen.shape[1]):
            n = int(chosen[t, c])
            y = h[t:t + 1] if n >= router["experts"] else bounded_unit(h[t:t + 1], w, f"{name}.e{n}", mlp["expert"]["limit"])
            out[t] += weight[t, c] * y[0]
    if mlp.get("shared"):
        out = out + bounded_unit(h, w, name + ".shared", mlp["shared"]["limit"])
    return out


MIXERS = {"attention": differential_attention, "attention_2": rotary_attention, "latent_attention": latent_attention}


def layers(config, w, tokens, dtype=torch.float64):
    """The residual stream after every layer, [layers, T, width], and the logits [T, vocab]."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = config["norm"]["eps"]
    x = w["embed"].to(dtype)[tokens] * config["embedding"]["scale"]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}"
        h = rms(x, eps) * w[p + ".norm1"].to(dtype)
        y = MIXERS[layer["type"]](h, w, p + ".mix", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + experts(h, w, p + ".mlp", layer["mlp"])
        x = x + y
        after.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"].to(dtype)) @ w["head"].to(dtype).T
    return torch.stack(after), logits


def forward(config, w, tokens, dtype=torch.float64):
    return layers(config, w, tokens, dtype)[1]
