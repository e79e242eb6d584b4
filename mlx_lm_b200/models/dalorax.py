"""Dalorax: a decoder-only model whose config.json lists its layers one by one.

The token embedding gets a fixed sinusoid of the position added (``parts.Sinusoidal``).  Every layer is a block over
a float32 residual stream with a Dynamic Tanh norm before and after each sublayer (``parts.SandwichBlock``,
``parts.DynamicTanh``): ``x += norm1b(mixer(norm1(x)))``, then ``x += norm2b(ff(norm2(x)))`` where the layer has a
feed-forward.  One kind of mixer:

``attention``   grouped-query attention without biases and without rotation, scores ``scale * q.k`` bounded by
                ``softcap * tanh(. / softcap)``, a sliding window of ``mask.size`` positions beside which the first
                ``mask.keep_first`` positions of the sequence stay visible, and a sigmoid gate per column of the
                concatenated heads (``parts.TalkingHeadsAttention`` with those options).  A layer whose mixer names
                ``kv_from: j`` has no key and value projections: it reads the pages of layer ``j``.

Feed-forwards: ``dense`` (``down(silu(gate x) * up x)``, ``parts.GatedMLP``) or ``moe`` (``parts.ExpertsMLP``: sigmoid
router scores, the ``top`` largest, their scores as weights on the experts' inputs).  The model's norm, then logits =
``logit_scale * embed x``.

config.json keys: ``architecture``, ``vocab``, ``width``, ``logit_scale``, ``norm.eps`` (unused by this norm), ``layers``
(``type``, ``mixer``: ``heads, kv_heads, dim, vdim, scale, softcap, mask.size, mask.keep_first`` and optionally ``kv_from``;
``mlp``: null, ``{kind: dense, ff}`` or ``{kind: moe, expert.ff, router.experts, router.top}``).  Tensor names: ``embed``,
``l<i>.norm1|norm1b|norm2|norm2b`` (+ ``.b``, ``.alpha``), ``l<i>.mix.q|k|v|g|o``, ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router`` and ``l<i>.mlp.e<n>.gate|up|down``, ``final.norm`` (+ ``.b``, ``.alpha``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.base import BaseModelArgs, ConfigError, _positive_int
from ..config.registry import register_architecture
from ..parts import (DynamicTanh, ExpertsMLP, GatedMLP, Init, ModelDescription, OutputHead, RunEntry, SandwichBlock,
                     Sinusoidal, TalkingHeadsAttention, TokenEmbedding)

SINUSOID_BASE = 10000.0


def _need(d, keys, what: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{what} must be an object with the keys {', '.join(keys)}")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{what} lacks required key(s): {', '.join(missing)}")


@dataclass
class ModelArgs(BaseModelArgs):
    architecture: str
    vocab: int
    width: int
    layers: list
    norm: dict = None
    logit_scale: float = 1.0

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        for i, spec in enumerate(self.layers):
            _need(spec, ["type", "mixer"], f"layers[{i}]")
            if spec["type"] != "attention":
                raise ConfigError(f"layers[{i}].type {spec['type']!r}: 'attention'")
            m, where = spec["mixer"], f"layers[{i}].mixer"
            _need(m, ["dim", "heads", "kv_heads", "mask", "scale", "vdim"], where)
            _need(m["mask"], ["size"], where + ".mask")
            for k in ("dim", "heads", "kv_heads", "vdim"):
                _positive_int(f"{where}.{k}", m[k])
            _positive_int(f"{where}.mask.size", m["mask"]["size"])
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{where}: {m['heads']} heads over {m['kv_heads']} key/value heads")
            src = m.get("kv_from")
            if src is not None:
                if not isinstance(src, int) or not 0 <= src < i:
                    raise ConfigError(f"{where}.kv_from {src!r}: an earlier layer's number")
                s = self.layers[src]["mixer"]
                if s.get("kv_from") is not None:
                    raise ConfigError(f"{where}.kv_from {src}: that layer has no keys and values of its own")
                if any(s[k] != m[k] for k in ("kv_heads", "dim", "vdim")):
                    raise ConfigError(f"{where}.kv_from {src}: the layers' key/value heads and sizes differ")
            mlp = spec.get("mlp")
            if mlp is not None:
                _need(mlp, ["kind"], f"layers[{i}].mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ["ff"], f"layers[{i}].mlp")
                elif mlp["kind"] == "moe":
                    _need(mlp, ["expert", "router"], f"layers[{i}].mlp")
                    _need(mlp["expert"], ["ff"], f"layers[{i}].mlp.expert")
                    _need(mlp["router"], ["experts", "top"], f"layers[{i}].mlp.router")
                    if not 1 <= mlp["router"]["top"] <= mlp["router"]["experts"]:
                        raise ConfigError(f"layers[{i}].mlp.router: top {mlp['router']['top']} of {mlp['router']['experts']}")
                else:
                    raise ConfigError(f"layers[{i}].mlp.kind {mlp['kind']!r}: 'dense' or 'moe'")

    @property
    def vocab_size(self) -> int:
        return self.vocab


def _norm(name: str, D: int, **kw) -> DynamicTanh:
    return DynamicTanh(name, D, bias=True, **kw)


def build(args: ModelArgs) -> ModelDescription:
    D = args.width
    lin = Init(0.0, D ** -0.5)
    embed = TokenEmbedding("embed", args.vocab, D, weight_suffix="", stream_dtype=torch.float32, init=Init(0.0, 1.0))
    # what the pages of a layer must keep: the widest window and the most kept first positions among the layers that
    # read them (the layer itself and those that name it in kv_from)
    owner = [spec["mixer"].get("kv_from") if spec["mixer"].get("kv_from") is not None else i
             for i, spec in enumerate(args.layers)]
    keep_window, keep_first = {}, {}
    for i, spec in enumerate(args.layers):
        mask = spec["mixer"]["mask"]
        keep_window[owner[i]] = max(keep_window.get(owner[i], 0), int(mask["size"]))
        keep_first[owner[i]] = max(keep_first.get(owner[i], 0), int(mask.get("keep_first", 0)))
    blocks, order = [], []
    for i, spec in enumerate(args.layers):
        p, m = f"l{i}", spec["mixer"]
        mixer = TalkingHeadsAttention(
            f"{p}.mix", D, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], 0.0, rot_dims=0, bias=False,
            talk=False, value_norm=False, head_gate=False, column_gate=True, window=int(m["mask"]["size"]),
            keep_first=int(m["mask"].get("keep_first", 0)), softcap=float(m.get("softcap") or 0.0),
            own_kv=owner[i] == i, cache_window=keep_window[owner[i]], cache_keep_first=keep_first[owner[i]], init=lin)
        norm_2 = ff = post_2 = None
        mlp = spec.get("mlp")
        if mlp is not None:
            norm_2, post_2 = _norm(f"{p}.norm2", D), _norm(f"{p}.norm2b", D)
            if mlp["kind"] == "dense":
                ff = GatedMLP(f"{p}.mlp", D, int(mlp["ff"]), init=lin)
            else:
                ff = ExpertsMLP(f"{p}.mlp", D, int(mlp["expert"]["ff"]), int(mlp["router"]["experts"]),
                                int(mlp["router"]["top"]), score="sigmoid", renormalize=False, scale_input=True, init=lin,
                                router_init=lin)
        blocks.append(SandwichBlock(_norm(f"{p}.norm1", D), mixer, _norm(f"{p}.norm1b", D), norm_2, ff, post_2))
        order.append(RunEntry(i, cache=owner[i], write=owner[i] == i))
    for a, b in zip(blocks, blocks[1:]):
        a.feeds = b          # a block's last stream update also leaves the next block's first norm
    return ModelDescription(
        model_type="dalorax", width=D, vocab_size=args.vocab, embedding=embed, position=Sinusoidal(D, SINUSOID_BASE),
        blocks=blocks, order=order, final_norm=_norm("final.norm", D, out_scale=float(args.logit_scale)),
        head=OutputHead(args.vocab, D, tied_to=embed), args=args)


register_architecture("dalorax", ModelArgs, build)
