"""Zuluvik: a decoder-only model whose config.json lists its layers one by one.

The token embedding is multiplied by ``embedding.scale``.  Every layer is a parallel block over a float32 residual
stream (``parts.ParallelBlock``): one RMS norm, whose output both the mixer and the feed-forward read, and
``x += mixer(h) + feed_forward(h)``.  Three kinds of mixer:

``attention``         two score maps per head over the same values, combined as a difference and normed per head
                      (``parts.DifferentialAttention``); q, k and v pass a short causal convolution of ``conv`` taps;
``attention_2``       grouped-query attention with biases on q, k and v, a rotation of the first ``rot.dims``
                      dimensions (pairs ``(2i, 2i+1)``), optionally stretched (``rot.scaling``), and q and k heads
                      divided by their root mean square after it (``parts.TalkingHeadsAttention`` with those options);
``latent_attention``  attention over latent rows ``[c | rotated key part]`` shared by all heads, the same kind of
                      rotation (``parts.LatentAttention``).

All are causal over the whole sequence.  The feed-forward (``mlp``, or null for none) is a mixture of experts
(``parts.ExpertsMLP``): softmax router scores over experts and identity experts together, a correction added for the
choice only, groups of which the best stay in the race, weights renormalised and scaled, experts with the bounded
gated unit, and a shared expert of the same form (``parts.GatedMLP``) that every token uses.

A layer with ``weights_of: j`` has no tensors: it runs layer ``j``'s block again, with a cache of its own.  The model's
RMS norm (``final.norm``), then logits = ``head x``.

config.json keys: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (``type``,
``mixer``, ``mlp``, ``weights_of``).  Mixer keys: ``heads, kv_heads, dim, vdim, scale`` and ``diff, conv`` (attention),
``rot`` (attention_2), ``heads, dim, rot_dim, vdim, kv_rank, scale, rot`` (latent_attention); ``rot``: ``base, dims`` and
optionally ``scaling`` (``factor, original, fast, slow``).  ``mlp``: ``kind: moe``, ``expert`` (``ff, limit``), ``router``
(``experts, top, identity, scale, groups.count, groups.keep``), ``shared`` (``ff, limit``).  Tensor names: ``embed``,
``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.router|correction``, ``l<i>.mlp.e<n>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..config.base import BaseModelArgs, ConfigError, _positive_int
from ..config.registry import register_architecture
from ..parts import (DifferentialAttention, ExpertsMLP, GatedMLP, Init, LatentAttention, ModelDescription, OutputHead,
                     ParallelBlock, RMSNorm, RunEntry, TalkingHeadsAttention, TokenEmbedding)

RENORMALIZE_EPS = 1e-20      # added to the sum the chosen experts' scores are divided by

MIXER_KEYS = {
    "attention": ["dim", "heads", "kv_heads", "scale", "vdim", "diff"],
    "attention_2": ["dim", "heads", "kv_heads", "scale", "vdim"],
    "latent_attention": ["dim", "heads", "kv_rank", "rot", "rot_dim", "scale", "vdim"],
}


def _need(d, keys, what: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{what} must be an object with the keys {', '.join(keys)}")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{what} lacks required key(s): {', '.join(missing)}")


def _check_rot(rot, where: str, most: int) -> None:
    _need(rot, ["base", "dims"], where)
    if not isinstance(rot["dims"], int) or rot["dims"] < 0 or rot["dims"] % 2 or rot["dims"] > most:
        raise ConfigError(f"{where}.dims {rot['dims']!r}: an even number up to {most}")
    if rot.get("scaling"):
        _need(rot["scaling"], ["factor", "original", "fast", "slow"], where + ".scaling")


@dataclass
class ModelArgs(BaseModelArgs):
    architecture: str
    vocab: int
    width: int
    layers: list
    norm: dict
    embedding: dict = field(default_factory=lambda: {"scale": 1.0})

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        _need(self.norm, ["eps"], "norm")
        _need(self.embedding, ["scale"], "embedding")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        for i, spec in enumerate(self.layers):
            _need(spec, ["type", "mixer"], f"layers[{i}]")
            if spec["type"] not in MIXER_KEYS:
                raise ConfigError(f"layers[{i}].type {spec['type']!r}: one of {sorted(MIXER_KEYS)}")
            m, where = spec["mixer"], f"layers[{i}].mixer"
            _need(m, MIXER_KEYS[spec["type"]], where)
            for k in ("dim", "heads", "vdim"):
                _positive_int(f"{where}.{k}", m[k])
            if spec["type"] == "latent_attention":
                _positive_int(f"{where}.kv_rank", m["kv_rank"])
                _check_rot(m["rot"], where + ".rot", m["rot_dim"])
                if m["rot"]["dims"] != m["rot_dim"]:
                    raise ConfigError(f"{where}: rot.dims {m['rot']['dims']} is not rot_dim {m['rot_dim']}")
            else:
                _positive_int(f"{where}.kv_heads", m["kv_heads"])
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}: {m['heads']} heads over {m['kv_heads']} key/value heads")
                if spec["type"] == "attention_2" and m.get("rot"):
                    _check_rot(m["rot"], where + ".rot", m["dim"])
            src = spec.get("weights_of")
            if src is not None:
                if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < len(self.layers) or src == i:
                    raise ConfigError(f"layers[{i}].weights_of {src!r}: another layer's number")
                other = self.layers[src]
                if other.get("weights_of") is not None:
                    raise ConfigError(f"layers[{i}].weights_of {src}: that layer has no tensors of its own")
                if any(other.get(k) != spec.get(k) for k in ("type", "mixer", "mlp")):
                    raise ConfigError(f"layers[{i}].weights_of {src}: the two layers' entries differ")
            mlp = spec.get("mlp")
            if mlp is not None:
                where = f"layers[{i}].mlp"
                _need(mlp, ["kind", "expert", "router"], where)
                if mlp["kind"] != "moe":
                    raise ConfigError(f"{where}.kind {mlp['kind']!r}: 'moe'")
                _need(mlp["expert"], ["ff", "limit"], where + ".expert")
                r = mlp["router"]
                _need(r, ["experts", "top"], where + ".router")
                outputs = r["experts"] + int(r.get("identity") or 0)
                if not 1 <= r["top"] <= outputs:
                    raise ConfigError(f"{where}.router: top {r['top']} of {outputs}")
                g = r.get("groups")
                if g:
                    _need(g, ["count", "keep"], where + ".router.groups")
                    if g["count"] < 1 or outputs % g["count"] or not 1 <= g["keep"] <= g["count"] \
                            or r["top"] > g["keep"] * (outputs // g["count"]):
                        raise ConfigError(f"{where}.router.groups: {outputs} router outputs in {g['count']} groups, "
                                          f"{g['keep']} kept, {r['top']} chosen")
                if mlp.get("shared"):
                    _need(mlp["shared"], ["ff", "limit"], where + ".shared")

    @property
    def vocab_size(self) -> int:
        return self.vocab


def _mixer(name: str, D: int, spec: dict, eps: float):
    m = spec["mixer"]
    lin = Init(0.0, D ** -0.5)
    if spec["type"] == "attention":
        return DifferentialAttention(name, D, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps, m["diff"],
                                     taps=int(m.get("conv") or 0), init=lin)
    if spec["type"] == "attention_2":
        rot = m.get("rot") or {"dims": 0, "base": 10000.0}
        return TalkingHeadsAttention(name, D, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps,
                                     rot_dims=int(rot["dims"]), rot_base=rot["base"], interleaved=True, bias=True,
                                     out_bias=False, talk=False, value_norm=False, head_gate=False, head_norm=True,
                                     rot_scaling=rot.get("scaling"), init=lin, bias_init=Init(0.0, 0.1))
    rot = m["rot"]
    return LatentAttention(name, D, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"], eps,
                           rot_base=rot["base"], interleaved=True, rot_scaling=rot.get("scaling"), init=lin)


def _feed_forward(name: str, D: int, mlp: dict):
    lin = Init(0.0, D ** -0.5)
    r, e = mlp["router"], mlp["expert"]
    shared = None
    if mlp.get("shared"):
        shared = GatedMLP(name + ".shared", D, int(mlp["shared"]["ff"]), init=lin, unit="bounded",
                          limit=float(mlp["shared"]["limit"]))
    g = r.get("groups")
    return ExpertsMLP(name, D, int(e["ff"]), int(r["experts"]), int(r["top"]), score="softmax", renormalize=True,
                      scale_input=False, init=lin, router_init=lin, correction=True,
                      groups=(int(g["count"]), int(g["keep"])) if g else None, identity=int(r.get("identity") or 0),
                      renormalize_eps=RENORMALIZE_EPS, weight_scale=float(r.get("scale", 1.0)), unit="bounded",
                      limit=float(e["limit"]), shared=shared)


def build(args: ModelArgs) -> ModelDescription:
    D, eps = args.width, float(args.norm["eps"])
    embed = TokenEmbedding("embed", args.vocab, D, scale=float(args.embedding["scale"]), weight_suffix="",
                           stream_dtype=torch.float32, init=Init(0.0, 1.0 / float(args.embedding["scale"])))
    blocks, block_of, order = [], {}, []
    for i, spec in enumerate(args.layers):
        if spec.get("weights_of") is not None:
            continue
        p = f"l{i}"
        ff = _feed_forward(f"{p}.mlp", D, spec["mlp"]) if spec.get("mlp") is not None else None
        block_of[i] = len(blocks)
        blocks.append(ParallelBlock(RMSNorm(f"{p}.norm1", D, eps), _mixer(f"{p}.mix", D, spec, eps), ff))
    # every layer has a cache of its own, numbered by the layer; a layer without tensors runs another layer's block
    n = len(blocks)
    for i, spec in enumerate(args.layers):
        src = spec.get("weights_of")
        b = block_of[i if src is None else src]
        order.append(RunEntry(b, cache=b if src is None else n + i, write=True))
    return ModelDescription(
        model_type="zuluvik", width=D, vocab_size=args.vocab, embedding=embed, position=None, blocks=blocks, order=order,
        final_norm=RMSNorm("final.norm", D, eps),
        head=OutputHead(args.vocab, D, name="head", weight_suffix="", init=Init(0.0, D ** -0.5)), args=args)


register_architecture("zuluvik", ModelArgs, build)
