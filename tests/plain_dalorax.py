"""A plain, slow Dalorax: whole sequences through straightforward torch code, one function per mechanism, written
from the design's equations and sharing nothing with the package.  ``weights``: tensor name -> tensor as stored."""
import math

import torch


def sinusoid(n, width, dtype):
    """Row p: column 2i = sin(p f_i), column 2i+1 = cos(p f_i), f_i = 10000^(-2i / width)."""
    p = torch.arange(n, dtype=torch.float64)[:, None]
    f = 10000.0 ** (-2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)[None, :]
    out = torch.zeros(n, width, dtype=torch.float64)
    out[:, 0::2] = torch.sin(p * f)
    out[:, 1::2] = torch.cos(p * f)[:, : width // 2]
    return out.to(dtype)


def dynamic_tanh(x, w, name):
    return torch.tanh(w[name + ".alpha"].to(x.dtype) * x) * w[name].to(x.dtype) + w[name + ".b"].to(x.dtype)


def visible(n, size, keep_first):
    """[i, j]: may position i read position j?"""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention(h, w, name, m, shared=None):
    """``shared``: the (keys, values) of the layer this one reads, or None for projections of its own.
    Returns (output, (keys, values))."""
    T, dt = h.shape[0], h.dtype
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[name + ".q"].to(dt).T).view(T, H, dk)
    if shared is None:
        k = (h @ w[name + ".k"].to(dt).T).view(T, G, dk)
        v = (h @ w[name + ".v"].to(dt).T).view(T, G, dv)
    else:
        k, v = shared
    see = visible(T, m["mask"]["size"], m["mask"].get("keep_first", 0))
    heads = []
    for a in range(H):
        c = a // (H // G)
        s = (q[:, a] @ k[:, c].T) * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        s = s.masked_fill(~see, -math.inf)
        heads.append(torch.softmax(s, dim=-1) @ v[:, c])
    o = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w[name + ".g"].to(dt).T)
    return o @ w[name + ".o"].to(dt).T, (k, v)


def gated_unit(h, w, name):
    dt = h.dtype
    g = h @ w[name + ".gate"].to(dt).T
    u = h @ w[name + ".up"].to(dt).T
    return (g * torch.sigmoid(g) * u) @ w[name + ".down"].to(dt).T


def route(h, w, name, top):
    """(weights [T, top], experts [T, top]): the largest sigmoid scores, as they are."""
    s = torch.sigmoid(h @ w[name + ".router"].to(h.dtype).T)
    return torch.topk(s, top, dim=-1)


def experts(h, w, name, mlp):
    weight, chosen = route(h, w, name, mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w[name + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for c in range(chosen.shape[1]):
            out[t] += gated_unit(weight[t, c] * h[t:t + 1], w, f"{name}.e{int(chosen[t, c])}")[0]
    return out


def layers(config, w, tokens, dtype=torch.float64):
    """The residual stream after every layer, [layers, T, width], and the logits [T, vocab]."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(dtype)[tokens] + sinusoid(len(tokens), config["width"], dtype)
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        src = m.get("kv_from")
        y, kept[i] = attention(dynamic_tanh(x, w, p + ".norm1"), w, p + ".mix", m, None if src is None else kept[src])
        x = x + dynamic_tanh(y, w, p + ".norm1b")
        mlp = layer.get("mlp")
        if mlp is not None:
            h = dynamic_tanh(x, w, p + ".norm2")
            y = gated_unit(h, w, p + ".mlp") if mlp["kind"] == "dense" else experts(h, w, p + ".mlp", mlp)
            x = x + dynamic_tanh(y, w, p + ".norm2b")
        after.append(x.clone())
    logits = (dynamic_tanh(x, w, "final.norm") @ w["embed"].to(dtype).T) * config.get("logit_scale", 1.0)
    return torch.stack(after), logits


def forward(config, w, tokens, dtype=torch.float64):
    return layers(config, w, tokens, dtype)[1]
