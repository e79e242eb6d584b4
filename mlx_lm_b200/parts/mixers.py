"""Token mixers.  ``Attention``: multi-head (or grouped-query) causal
attention over a paged key/value cache.

One fused projection gives ``[q | k | v]`` per token (q = the first
``n_heads*head_dim`` columns, then k, then v, head j = columns
``[j*head_dim, (j+1)*head_dim)`` of each: mlx_lm/models/gpt2.py:52-58).  This
step's keys and values go into the request's pages first, then every token
attends keys ``max(0, p-window+1) .. p`` of its request through the block
table with scale ``head_dim**-0.5`` (mlx_lm/models/gpt2.py:39, 63-65), and
the output projection adds the residual in its epilogue.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import MATRIX, VECTOR, Init, Mixer, Normed, PagedKVSpec, ParamSpec, PositionEncoding, StateSpec, register_part
from .linear import FusedLinear, Linear
from .positions import rotation_frequencies


class Attention(Mixer):
    replayable = True
    kernel_libs = ("attention", "attention_prefill", "attention_prefill_tc")

    def __init__(self, name: str, width: int, n_heads: int, head_dim: int, n_kv_heads: Optional[int] = None,
                 window: Optional[int] = None, bias: bool = True, stored: str = "out_in",
                 qkv_name: str = "c_attn", out_name: str = "c_proj", scale: Optional[float] = None,
                 position: Optional[PositionEncoding] = None, init: Init = Init(), bias_init: Init = Init()):
        n_kv_heads = n_heads if n_kv_heads is None else n_kv_heads
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"{name}: head size {head_dim} must be a multiple of 16 between 16 and 256")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.head_dim, self.window = n_heads, n_kv_heads, head_dim, window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.position = position
        self.q_width, self.kv_width = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv = Linear(f"{name}.{qkv_name}", width, self.q_width + 2 * self.kv_width, bias, stored,
                          init=init, bias_init=bias_init)
        self.out = Linear(f"{name}.{out_name}", self.q_width, width, bias, stored, init=init, bias_init=bias_init)

    def children(self):
        return (self.qkv, self.out)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def fold_input_norm(self, norm) -> bool:
        return self.qkv.fold_norm(norm)

    def forward(self, ctx, x, residual, cache):
        T = x.shape[0]
        qkv = ctx.ws.get("qkv", T, self.q_width + 2 * self.kv_width, x.dtype)
        q = qkv[:, :self.q_width]
        src = x.source if isinstance(x, Normed) else x      # a Normed: the norm is folded into the projection
        if (cache.write and self.position is None and x.dtype == torch.bfloat16 and self.width % 8 == 0
                and src.stride(0) % 8 == 0 and src.data_ptr() % 16 == 0):
            # nothing to do to q and k before the cache: the projection's epilogue puts keys and values
            # into the pages itself
            fold = self.qkv.fold_of(ctx, x, few=T <= ops.SMALL_M) if isinstance(x, Normed) else None
            n_qkv = self.q_width + 2 * self.kv_width
            ops.label(self.qkv.name, 2.0 * T * self.width * n_qkv,
                      x.dtype.itemsize * (self.width * n_qkv + T * self.width + T * n_qkv))
            ops.linear_qkv_to_cache(src, self.qkv.weight, self.qkv.bias, qkv, ctx.positions, ctx.token_req,
                                    cache.block_table, cache.k, cache.v, self.q_width, ctx.status, ctx.stream,
                                    fold=fold)
        else:
            self.qkv.forward(ctx, x, qkv)
            k = qkv[:, self.q_width:self.q_width + self.kv_width]
            v = qkv[:, self.q_width + self.kv_width:]
            if self.position is not None:
                self.position.rotate(ctx, q, k)
            if cache.write:
                ops.kv_write(k, v, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, ctx.status,
                             ctx.stream)
        o = ctx.ws.get("attn_out", T, self.q_width, x.dtype)
        ops.label(self.name + ".attention")      # its cost depends on the requests' lengths: the caller knows them
        self.attend(ctx, q, cache, o)
        return self.out.forward(ctx, o, residual, residual=residual)

    def attend(self, ctx, q, cache, o) -> None:
        paged_attention(ctx, q, cache, o, self.n_heads, self.head_dim, self.scale, self.window)


def paged_attention(ctx, q, cache, o, n_heads: int, head_dim: int, scale: float, window: Optional[int],
                    sinks=None) -> None:
    """Causal attention of this step's queries over their requests' pages.  Rows of requests that bring one token
    go to a kernel for single queries (on tensor cores in bfloat16 for head sizes that are multiples of 16 up to
    128, else the split-key kernel on the CUDA cores), the rest to the kernel for portions; all write their rows
    of ``o``.  ``sinks``: float32 ``[n_heads]``, one more term of each head's softmax denominator, or None."""
    window = window or 0
    single_tiles = getattr(ctx, "single_tiles", None)
    if (ctx.n_single and single_tiles is not None
            and ops.attention_rows_supported(q.dtype, head_dim, ctx.n_single, n_heads, scale)):
        ops.attention_rows(q, single_tiles, ctx.n_single, cache.block_table, cache.k, cache.v, o, n_heads,
                           scale, window, ctx.status, ctx.stream, sinks=sinks)
    elif ctx.n_single:
        scratch = ctx.ws.flat("attn_partial", ops.attention_decode_scratch(
            ctx.n_single, n_heads, head_dim, ctx.max_len), torch.float32)
        counters = ctx.ws.flat("attn_tickets", ctx.n_single * n_heads, torch.int32)
        ops.attention_decode(q, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, o,
                             n_heads, scale, window, scratch, counters, ctx.max_len, ctx.status,
                             ctx.stream, rows=ctx.single_rows, sinks=sinks)
    if ctx.n_portion:
        if ops.attention_portions_supported(q.dtype, head_dim, scale) and ctx.portion_tiles is not None:
            ops.attention_portions(q, ctx.portion_tiles, ctx.n_portion_tiles, cache.block_table, cache.k,
                                   cache.v, o, n_heads, scale, window, ctx.status, ctx.stream, sinks=sinks,
                                   first_positions=ctx.req_first_position)
        else:
            ops.attention_generic(q, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, o,
                                  n_heads, scale, window, ctx.status, ctx.stream,
                                  rows=ctx.portion_rows, sinks=sinks)


register_part("mixer", "attention", Attention)


class SinkAttention(Mixer):
    """Grouped-query causal attention with the options of recent designs, each a parameter:

    * separate ``q``, ``k``, ``v`` tensors (run as one product), key/query size ``dim`` and value size ``vdim``
      that may differ (the pages hold heads ``head_dim`` wide, zero-filled beyond a head's own size);
    * ``qk_norm``: an RMS norm over a token's whole q projection, and whole k projection, before the heads are
      split, with plain weights ``<name>.q.norm`` / ``<name>.k.norm``;
    * ``rot_dims``: the first so many dimensions of every head turn with the position (dimension ``i`` paired
      with ``i + rot_dims/2``, angle ``p * rot_base**(-2i/rot_dims)``); 0 = no rotation;
    * ``scale`` of the scores as given; ``sink``: a learned number per head (``<name>.sink``) whose exponential
      is one more term of the softmax denominator, without a key or a value; ``window`` as in ``Attention``.

    ``mix`` returns the output projection in float32 (for a caller that combines it with something else);
    ``forward`` adds it to a float32 residual stream in that projection's epilogue."""
    replayable = True
    kernel_libs = ("attention", "attention_prefill", "attention_prefill_tc", "rotary")

    def __init__(self, name: str, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, rot_dims: int = 0, rot_base: float = 10000.0, qk_norm: bool = True, sink: bool = True,
                 window: Optional[int] = None, init: Init = Init()):
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"{name}: {rot_dims} rotated dimensions of {dim}")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.dim, self.vdim = n_heads, n_kv_heads, dim, vdim
        self.head_dim = (max(dim, vdim) + 15) // 16 * 16
        if self.head_dim > 256:
            raise ValueError(f"{name}: head size {max(dim, vdim)} is beyond 256")
        self.scale, self.eps, self.window = float(scale), float(eps), window
        self.rot_dims, self.rot_base, self.qk_norm, self.has_sink = rot_dims, float(rot_base), qk_norm, sink
        self.qkv = FusedLinear(f"{name}.qkv", width, [(f"{name}.q", n_heads * dim), (f"{name}.k", n_kv_heads * dim),
                                                      (f"{name}.v", n_kv_heads * vdim)], init=init)
        self.out = Linear(f"{name}.o", n_heads * vdim, width, bias=False, weight_suffix="", init=init)
        self.q_norm = self.k_norm = self.sinks = self.freq = None

    def children(self):
        return (self.qkv, self.out)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def param_specs(self) -> List[ParamSpec]:
        specs = []
        if self.qk_norm:
            specs += [ParamSpec(f"{self.name}.q.norm", (self.n_heads * self.dim,), VECTOR, Init(1.0, 0.1)),
                      ParamSpec(f"{self.name}.k.norm", (self.n_kv_heads * self.dim,), VECTOR, Init(1.0, 0.1))]
        if self.has_sink:
            specs.append(ParamSpec(f"{self.name}.sink", (self.n_heads,), VECTOR, Init(0.0, 1.0)))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        if self.qk_norm:
            self.q_norm, self.k_norm = tensors[f"{self.name}.q.norm"], tensors[f"{self.name}.k.norm"]
        if self.has_sink:
            self.sinks = tensors[f"{self.name}.sink"]
        if self.rot_dims:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.freq = (self.rot_base ** (-2.0 * i / self.rot_dims)).to(torch.float32).to(device)

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        if self.head_dim != self.vdim:
            # the attention kernels leave heads head_dim wide: give the output projection zero columns there
            w = self.out.weight.view(self.width, self.n_heads, self.vdim)
            wide = torch.zeros(self.width, self.n_heads, self.head_dim, dtype=w.dtype, device=w.device)
            wide[:, :, :self.vdim] = w
            self.out.use_weight(wide.view(self.width, self.n_heads * self.head_dim).contiguous())
            self.out.n_in = self.n_heads * self.head_dim

    def _heads_out(self, ctx, x, cache):
        T, H, G = x.shape[0], self.n_heads, self.n_kv_heads
        n = self.qkv.n_out
        proj = ctx.ws.get("attn_proj", T, (n + 7) // 8 * 8, x.dtype)[:, :n]
        self.qkv.forward(ctx, x, proj)
        q = ctx.ws.get("attn_q", T, H * self.head_dim, x.dtype)
        ops.label(self.name + ".prepare", 8.0 * T * n, 2.0 * x.element_size() * T * n)
        ops.qkv_prepare(proj, 0, H * self.dim, (H + G) * self.dim, H, G, self.dim, self.vdim, self.q_norm, self.k_norm,
                        self.eps, self.freq, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, q,
                        cache.write, ctx.status, ctx.stream)
        o = ctx.ws.get("attn_out", T, H * self.head_dim, x.dtype)
        ops.label(self.name + ".attention")
        paged_attention(ctx, q, cache, o, H, self.head_dim, self.scale, self.window, sinks=self.sinks)
        return o

    def mix(self, ctx, x, cache, tag: str = "mix_left"):
        o = self._heads_out(ctx, x, cache)
        return self.out.forward(ctx, o, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._heads_out(ctx, x, cache), residual, residual=residual)


class ParallelMixer(Mixer):
    """Two mixers side by side on the same input: ``scale * (norm_l(left(x)) + norm_r(right(x)))`` added to the
    residual stream, each output RMS-normed over the model width with a plain weight (``<name>.left.out`` /
    ``<name>.right.out``) first.  Each side keeps its own cache (``cache_spec`` is a dictionary); the sides are
    any mixers that have ``mix(ctx, x, cache, tag) -> float32 [T, width]``."""
    replayable = True
    kernel_libs = ("rms",)

    def __init__(self, name: str, width: int, left: Mixer, right: Mixer, eps: float, scale: float = 0.5):
        self.name, self.width, self.left, self.right, self.eps, self.scale = name, width, left, right, float(eps), scale
        self.w_left = self.w_right = None

    def children(self):
        return (self.left, self.right)

    def cache_spec(self):
        out = {}
        for side, m in (("left", self.left), ("right", self.right)):
            spec = m.cache_spec()
            if isinstance(spec, dict):
                out.update({f"{side}.{k}": v for k, v in spec.items()})
            elif spec is not None:
                out[side] = spec
        return out

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(f"{self.name}.left.out", (self.width,), VECTOR, Init(1.0, 0.1)),
                ParamSpec(f"{self.name}.right.out", (self.width,), VECTOR, Init(1.0, 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        self.w_left, self.w_right = tensors[f"{self.name}.left.out"], tensors[f"{self.name}.right.out"]

    def forward(self, ctx, x, residual, cache):
        yl = self.left.mix(ctx, x, cache.side("left"), tag="mix_left")
        yr = self.right.mix(ctx, x, cache.side("right"), tag="mix_right")
        ops.label(self.name + ".combine", 8.0 * x.shape[0] * self.width, 16.0 * x.shape[0] * self.width)
        ops.residual_update(residual, yl, ctx.stream, w1=self.w_left, y2=yr, w2=self.w_right, scale=self.scale,
                            eps=self.eps)
        return residual


def visible_pairs(ctx, window: Optional[int], chunk: Optional[int]):
    """For a label: how many (query, key) pairs this step's queries see, and how many distinct keys they read."""
    pairs = keys = 0
    for sp in ctx.spans:
        first = None
        for p in range(sp.first_position, sp.first_position + sp.n_tokens):
            lo = max(0, p - window + 1) if window else 0
            if chunk:
                lo = max(lo, p // chunk * chunk)
            pairs += p - lo + 1
            first = lo if first is None else min(first, lo)
        keys += sp.first_position + sp.n_tokens - (first or 0)
    return pairs, keys


class TalkingHeadsAttention(Mixer):
    """Grouped-query causal attention in which a CTA of the attention kernel takes all heads of a query
    (``ops.attention_wide``), with these options, each a parameter:

    * separate ``q``, ``k``, ``v`` tensors with biases ``<tensor>.b`` (``bias``), run as one product together
      with the gate's; key/query size ``dim`` and value size ``vdim`` may differ;
    * ``rot_dims``: the first so many dimensions of every q and k head turn with the position, angle
      ``p * rot_base**(-2i/rot_dims)``, pairs ``(i, i + rot_dims/2)`` or, ``interleaved``, ``(2i, 2i+1)``;
      ``rot_scaling`` (``factor``, ``original``, ``fast``, ``slow``) stretches the slow pairs and puts a factor on
      cosine and sine (``parts.rotation_frequencies``);
    * ``head_norm``: every q and k head is divided by its root mean square over ``dim`` after the rotation (eps inside
      the root, no weight);
    * ``out_bias``: whether ``<name>.o`` has a bias (default: as the other projections);
    * ``value_norm``: every value head is divided by its root mean square (eps inside the root, no weight)
      before it enters the cache;
    * ``talk``: the heads' scores ``scale * q_g . k`` are mixed before the softmax, ``s_h <- sum_g T[h, g] s_g``
      with ``T`` = ``<name>.talk`` ``[heads, heads]``;
    * ``window``: position ``p`` sees the last ``window`` positions; ``chunk``: it sees ``j <= p`` of its own run of
      ``chunk`` positions, runs counted from position 0 of the sequence (earlier runs' pages are given back);
    * ``head_gate``: head ``h``'s output times ``sigmoid(W_g x)_h`` (``<name>.g`` ``[heads, width]``, the mixer's own
      input), before the output projection ``<name>.o`` (bias ``<name>.o.b``); ``column_gate``: every column of the
      concatenated heads has a gate of its own (``<name>.g`` ``[heads * vdim, width]``);
    * ``softcap``: scores become ``softcap * tanh(score / softcap)`` after the scale, before the softmax;
    * ``keep_first``: beside the window, the first ``keep_first`` positions of the sequence stay visible to every later
      position (``j <= p and (p - j < window or j < keep_first)``); their pages are never given back;
    * ``own_kv=False``: the layer has no key and value projections; it reads the pages another layer wrote (the run
      order points it there with ``write=False``) with its own queries, mask, scale and gate.  ``cache_window`` and
      ``cache_keep_first`` say what the shared pages must keep when the layers that read them differ in their masks
      (by default this layer's own ``window`` and ``keep_first``); all layers on one cache give the same.

    Queries go to the kernel in float32; scores, their mix and the softmax are float32.  ``mix`` returns the output
    projection in float32 for a block that adds it to the stream itself; ``forward`` adds it in that product's epilogue."""
    replayable = True
    kernel_libs = ("attention_wide", "attention_wide_tc", "rotary")

    def __init__(self, name: str, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, rot_dims: int = 0, rot_base: float = 10000.0, interleaved: bool = False, bias: bool = True,
                 talk: bool = True, value_norm: bool = True, head_gate: bool = True, window: Optional[int] = None,
                 chunk: Optional[int] = None, init: Init = Init(), bias_init: Init = Init(), column_gate: bool = False,
                 softcap: float = 0.0, keep_first: int = 0, own_kv: bool = True, cache_window: Optional[int] = None,
                 cache_keep_first: Optional[int] = None, rot_scaling: Optional[dict] = None, head_norm: bool = False,
                 out_bias: Optional[bool] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"{name}: {rot_dims} rotated dimensions of {dim}")
        if not own_kv and head_norm:
            raise ValueError(f"{name}: a layer that reads another layer's pages does not norm their keys")
        self.rot_scaling, self.head_norm, self.rot_mscale = rot_scaling, head_norm, 1.0
        if head_gate and column_gate:
            raise ValueError(f"{name}: a gate per head or a gate per column, not both")
        if keep_first and not window:
            raise ValueError(f"{name}: kept first positions go with a window")
        if not own_kv and (value_norm or rot_dims):
            raise ValueError(f"{name}: a layer that reads another layer's pages neither rotates nor norms them")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.dim, self.vdim = n_heads, n_kv_heads, dim, vdim
        self.column_gate, self.softcap, self.keep_first, self.own_kv = column_gate, float(softcap or 0.0), int(keep_first or 0), own_kv
        self.cache_window = window if cache_window is None else cache_window
        self.cache_keep_first = self.keep_first if cache_keep_first is None else int(cache_keep_first)
        self.key_row, self.value_row = (dim + 7) // 8 * 8, (vdim + 7) // 8 * 8     # rows of the pages: whole 16 bytes
        self.scale, self.eps, self.window, self.chunk = float(scale), float(eps), window, chunk
        self.rot_dims, self.rot_base, self.interleaved = rot_dims, float(rot_base), interleaved
        self.has_talk, self.value_norm, self.head_gate = talk, value_norm, head_gate
        sources = [(f"{name}.q", n_heads * dim)]
        if own_kv:
            sources += [(f"{name}.k", n_kv_heads * dim), (f"{name}.v", n_kv_heads * vdim)]
        biases = {n: n + ".b" for n, _ in sources} if bias else None
        if head_gate or column_gate:
            sources.append((f"{name}.g", n_heads * vdim if column_gate else n_heads))
        self.proj = FusedLinear(f"{name}.qkvg", width, sources, init=init, biases=biases, bias_init=bias_init)
        self.out = Linear(f"{name}.o", n_heads * vdim, width, bias=False, weight_suffix="", init=init)
        self.has_bias, self.bias_init = bias, bias_init
        self.has_out_bias = bias if out_bias is None else bool(out_bias)
        self.talk = self.freq = None
        if dim == 64 and vdim == 64 and not talk and not chunk and not head_gate:
            # plain heads of 64: prompt portions run on the tcgen05 kernel (queries that were turned or normed reach it
            # through a bfloat16 copy)
            self.kernel_libs = type(self).kernel_libs + ("attention_prefill_tc", "elementwise")

    def children(self):
        return (self.proj, self.out)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.key_row, self.cache_window, chunk=self.chunk, value_dim=self.value_row,
                           keep_first=self.cache_keep_first or None)

    def param_specs(self) -> List[ParamSpec]:
        specs = []
        if self.has_talk:
            specs.append(ParamSpec(f"{self.name}.talk", (self.n_heads, self.n_heads), VECTOR, Init(0.0, 0.5)))
        if self.has_out_bias:
            specs.append(ParamSpec(f"{self.name}.o.b", (self.width,), VECTOR, self.bias_init))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        if self.has_talk:
            self.talk = tensors[f"{self.name}.talk"].contiguous()
        if self.rot_dims:
            f, self.rot_mscale = rotation_frequencies(self.rot_dims, self.rot_base, self.rot_scaling)
            self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        if self.has_out_bias:
            self.out.bias = tensors[f"{self.name}.o.b"]     # named beside the tensor, not ".bias": set once the layer is bound

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._heads_out(ctx, x, cache), residual, residual=residual)

    def mix(self, ctx, x, cache, tag: str = "mix_out"):
        o = self._heads_out(ctx, x, cache)
        return self.out.forward(ctx, o, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def _heads_out(self, ctx, x, cache):
        T, H, G = x.shape[0], self.n_heads, self.n_kv_heads
        if cache.write != self.own_kv:
            raise ops.KernelError(f"{self.name}: a layer {'with' if self.own_kv else 'without'} key and value "
                                  f"projections {'writes its' if self.own_kv else 'only reads another layer\'s'} pages")
        n = self.proj.n_out
        proj = ctx.ws.get("attn_proj", T, (n + 7) // 8 * 8, x.dtype)[:, :n]
        self.proj.forward(ctx, x, proj)
        q = ctx.ws.get("attn_q32", T, H * self.key_row, torch.float32)
        ops.label(self.name + ".prepare", 8.0 * T * n, (x.element_size() + 4.0) * T * n)
        self._prepare(ctx, proj, cache, q)
        # without a rotation (and without a norm of the heads) the product's own (rounded) query columns are the queries
        q_rounded = proj[:, :H * self.dim] if not self.rot_dims and not self.head_norm and proj.dtype == cache.k.dtype else None
        if (q_rounded is None and ctx.n_portion and ctx.portion_tiles is not None and "attention_prefill_tc" in self.kernel_libs
                and proj.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16 and ops.PREFILL_TC):
            # turned or normed queries of plain heads of 64: the tcgen05 kernel for portions takes them in bfloat16
            q_rounded = ctx.ws.get("attn_q16", T, H * self.key_row, torch.bfloat16)
            ops.label(self.name + ".prepare.cast", 0.0, 6.0 * T * H * self.key_row)
            ops.join_rows(q, None, q_rounded, ctx.stream)
        o = ctx.ws.get("attn_out", T, H * self.vdim, x.dtype)
        if ops.recording():
            pairs, keys = visible_pairs(ctx, self.window, self.chunk)
            ops.label(self.name + ".attention", pairs * H * (2.0 * self.dim + 2.0 * self.vdim + 2.0 * H),
                      x.element_size() * (keys * G * (self.key_row + self.value_row) + T * H * self.vdim) + 4.0 * T * H * self.dim)
        gate = None
        if self.head_gate or self.column_gate:
            g_off = self.proj.offset(f"{self.name}.g")
            gate = proj[:, g_off:g_off + (H * self.vdim if self.column_gate else H)]
        ops.attention_wide_step(ctx, q, self.key_row, cache.k, cache.v, cache.block_table, o, self.vdim, H, self.dim,
                                self.vdim, self.scale, window=self.window or 0, chunk=self.chunk or 0, talk=self.talk,
                                gate=gate, softcap=self.softcap, keep_first=self.keep_first, q_rounded=q_rounded)
        return o

    def _prepare(self, ctx, proj, cache, q) -> None:
        H, G = self.n_heads, self.n_kv_heads
        # (a layer without key and value projections passes offsets that are never read: nothing is written)
        ops.qkv_prepare(proj, 0, H * self.dim, (H + G) * self.dim, H, G, self.dim, self.vdim, None, None, self.eps,
                        self.freq, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, q, cache.write,
                        ctx.status, ctx.stream, interleaved=self.interleaved,
                        v_norm_eps=self.eps if self.value_norm else None, mscale=self.rot_mscale,
                        head_norm_eps=self.eps if self.head_norm else None)


class LatentAttention(Mixer):
    """Attention whose keys and values of all heads are kept as one short latent row per token.

    ``<name>.q`` gives every head ``[dim unrotated | rot_dim rotated]`` query dimensions; ``<name>.dkv`` gives
    ``kv_rank`` latent columns, RMS-normed with the weight ``<name>.dkv.norm`` (``c``), and ``rot_dim`` columns of a
    rotated key part that all heads share.  Head ``h``'s unrotated key is ``W_uk_h c`` (``<name>.uk``) and its value
    ``W_uv_h c`` (``<name>.uv``); its score is ``scale * (q_unrotated . k_unrotated + q_rotated . k_rotated)``.

    The pages hold ``[c | rotated key part]`` only (one row per token, no value pool).  The keys' up-projection
    is applied to the queries instead (``q_h -> W_uk_h^T q_h``, a product per head), the attention runs over the latent
    rows with all heads sharing them (the values are the rows' first ``kv_rank`` columns), and the values'
    up-projection is applied to its output (again a product per head), then ``<name>.o``.  Queries and the
    attention's output stay float32 between those products.  Rotation pairs ``(2i, 2i+1)`` (``interleaved``) or
    ``(i, i + rot_dim/2)``, optionally stretched (``rot_scaling``, see ``parts.rotation_frequencies``; the scores' scale
    stays as given); ``window`` as in the other attention parts."""
    replayable = True
    kernel_libs = ("attention_wide", "attention_wide_tc", "latent")

    def __init__(self, name: str, width: int, n_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, eps: float, rot_base: float = 10000.0, interleaved: bool = True,
                 window: Optional[int] = None, chunk: Optional[int] = None, init: Init = Init(),
                 rot_scaling: Optional[dict] = None):
        if rot_dim % 2:
            raise ValueError(f"{name}: {rot_dim} rotated dimensions")
        self.rot_scaling, self.rot_mscale = rot_scaling, 1.0
        self.name, self.width = name, width
        self.n_heads, self.dim, self.rot_dim, self.vdim, self.rank = n_heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.window, self.chunk = float(scale), float(eps), window, chunk
        self.rot_base, self.interleaved = float(rot_base), interleaved
        self.q_head = dim + rot_dim
        self.lat = kv_rank + rot_dim                      # what a score is taken over
        self.row = (self.lat + 7) // 8 * 8                # a page row: whole 16 bytes
        self.proj = FusedLinear(f"{name}.q_dkv", width, [(f"{name}.q", n_heads * self.q_head),
                                                         (f"{name}.dkv", kv_rank + rot_dim)], init=init)
        self.out = Linear(f"{name}.o", n_heads * vdim, width, bias=False, weight_suffix="", init=init)
        self.init = init
        self.norm_w = self.w_absorb = self.w_values = self.freq = None

    def children(self):
        return (self.proj, self.out)

    def cache_spec(self):
        return PagedKVSpec(1, self.row, self.window, chunk=self.chunk, value_dim=0)

    def param_specs(self) -> List[ParamSpec]:
        n, H, R = self.name, self.n_heads, self.rank
        up = Init(0.0, R ** -0.5)
        return [ParamSpec(f"{n}.dkv.norm", (R,), VECTOR, Init(1.0, 0.1)),
                ParamSpec(f"{n}.uk", (H * self.dim, R), MATRIX, up),
                ParamSpec(f"{n}.uv", (H * self.vdim, R), MATRIX, up)]

    def bind(self, tensors, dtype, device) -> None:
        n, H, R = self.name, self.n_heads, self.rank
        self.norm_w = tensors[f"{n}.dkv.norm"]
        # [H, rank, dim]: head h's matrix from its unrotated query to the latent columns
        self.w_absorb = tensors[f"{n}.uk"].view(H, self.dim, R).transpose(1, 2).contiguous()
        self.w_values = tensors[f"{n}.uv"].view(H, self.vdim, R).contiguous()
        if self.rot_dim:
            f, self.rot_mscale = rotation_frequencies(self.rot_dim, self.rot_base, self.rot_scaling)
            self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)

    def forward(self, ctx, x, residual, cache):
        T, H, R = x.shape[0], self.n_heads, self.rank
        n = self.proj.n_out
        proj = ctx.ws.get("latent_proj", T, (n + 7) // 8 * 8, x.dtype)[:, :n]
        self.proj.forward(ctx, x, proj)
        q_lat = ctx.ws.get("latent_q", T, H * self.lat, torch.float32)
        ops.label(self.name + ".prepare", 8.0 * T * n, x.element_size() * T * (n + self.row) + 4.0 * T * H * self.rot_dim)
        ops.latent_prepare(proj, 0, H * self.q_head, H, self.dim, self.rot_dim, R, self.norm_w, self.eps, self.freq,
                           self.interleaved, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.write, q_lat,
                           self.lat, ctx.status, ctx.stream, mscale=self.rot_mscale)
        ops.label(self.name + ".uk", 2.0 * T * H * self.dim * R, x.element_size() * (T * H * self.dim + H * self.dim * R)
                  + 4.0 * T * H * R)
        ops.head_linear(proj, self.q_head, self.w_absorb, q_lat, self.lat, ctx.stream, token_req=ctx.token_req)
        o_lat = ctx.ws.get("latent_o", T, H * R, torch.float32)
        if ops.recording():
            pairs, keys = visible_pairs(ctx, self.window, self.chunk)
            ops.label(self.name + ".latent.attention", pairs * H * 2.0 * (self.lat + R),
                      x.element_size() * keys * self.row + 4.0 * T * H * (self.lat + R))
        ops.attention_wide_step(ctx, q_lat, self.lat, cache.k, cache.k, cache.block_table, o_lat, R, H, self.lat, R,
                                self.scale, window=self.window or 0, chunk=self.chunk or 0)
        o = ctx.ws.get("attn_out", T, H * self.vdim, x.dtype)
        ops.label(self.name + ".uv", 2.0 * T * H * self.vdim * R, 4.0 * T * H * R + x.element_size() * (H * self.vdim * R
                  + T * H * self.vdim))
        ops.head_linear(o_lat, R, self.w_values, o, self.vdim, ctx.stream, token_req=ctx.token_req)
        return self.out.forward(ctx, o, residual, residual=residual)


class DifferentialAttention(Mixer):
    """Grouped-query causal attention with two score maps per head over the same values.

    ``<name>.q`` gives every query head ``[map 1 | map 2]`` (``2 * dim`` columns), ``<name>.k`` every key head the
    same, ``<name>.v`` every key/value head ``vdim`` columns; no biases, no rotation.  With ``taps`` > 0 each channel
    of q, k and v passes a short causal convolution over time right after the projection (``<tensor>.conv``
    ``[channels, taps]``, last column: the current token; no bias, no activation) whose last ``taps - 1`` inputs are
    part of the request's state.  Each map is an ordinary softmax attention ``a_m`` with scores ``scale * q_m . k_m``;
    a head's output is ``o = a_1 - lambda a_2`` with one number for the layer,
    ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (``<name>.lq1`` and so on, ``dim`` values each), then ``o``
    divided by its root mean square over ``vdim`` (eps inside the root, no weight) and multiplied by ``1 - diff``,
    then ``<name>.o``.

    The pages hold ``2 * kv_heads`` key heads (a key head's two maps side by side) and ``kv_heads`` value heads
    (``PagedKVSpec.value_heads``); the attention kernels run ``2 * heads`` independent query heads, ordered (when the
    weights are bound, by a permutation of the rows of ``q`` and of its convolution) so that the queries of one key
    head lie together: group ``g`` holds ``[map 1 of its heads | map 2 of its heads]``."""
    replayable = True
    kernel_libs = ("attention_wide", "attention_wide_tc", "rotary", "recurrent", "rms")

    def __init__(self, name: str, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, diff: float, taps: int = 0, init: Init = Init()):
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if taps < 0 or taps > 9:
            raise ValueError(f"{name}: a convolution of {taps} taps (at most 9)")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.dim, self.vdim = n_heads, n_kv_heads, dim, vdim
        self.scale, self.eps, self.diff, self.taps = float(scale), float(eps), float(diff), int(taps or 0)
        self.key_row, self.value_row = (dim + 7) // 8 * 8, (vdim + 7) // 8 * 8
        self.q_width, self.k_width, self.v_width = n_heads * 2 * dim, n_kv_heads * 2 * dim, n_kv_heads * vdim
        self.conv_width = self.q_width + self.k_width + self.v_width
        self.proj = FusedLinear(f"{name}.qkv", width, [(f"{name}.q", self.q_width), (f"{name}.k", self.k_width),
                                                       (f"{name}.v", self.v_width)], init=init)
        self.out = Linear(f"{name}.o", n_heads * vdim, width, bias=False, weight_suffix="", init=init)
        self.lam = 0.0
        self.conv_w = self.conv_wt = self._no_state = None
        if dim == 64 and vdim % 64 == 0:
            # maps of 64 over values of 64 or a multiple: prompt portions run on the tcgen05 kernel
            self.kernel_libs = type(self).kernel_libs + ("attention_prefill_tc", "elementwise")

    def children(self):
        return (self.proj, self.out)

    def cache_spec(self):
        kv = PagedKVSpec(2 * self.n_kv_heads, self.key_row, None, value_dim=self.value_row, value_heads=self.n_kv_heads)
        if self.taps > 1:
            return {"kv": kv, "conv": StateSpec((self.taps - 1, self.conv_width))}
        return kv

    def param_specs(self) -> List[ParamSpec]:
        n = self.name
        specs = []
        if self.taps:
            specs += [ParamSpec(f"{n}.{t}.conv", (w, self.taps), VECTOR, Init(0.0, 0.4))
                      for t, w in (("q", self.q_width), ("k", self.k_width), ("v", self.v_width))]
        specs += [ParamSpec(f"{n}.{t}", (self.dim,), VECTOR, Init(0.0, 0.1)) for t in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def _query_order(self, device) -> torch.Tensor:
        """Rows of the stored ``q`` in the order the kernels want them: blocks of ``dim`` rows, block ``(g, m, r)`` (key
        head, map, query head of the group) taken from the stored block ``(g * rep + r, m)``."""
        H, G, d = self.n_heads, self.n_kv_heads, self.dim
        rep = H // G
        blocks = [(g * rep + r) * 2 + m for g in range(G) for m in range(2) for r in range(rep)]
        idx = torch.tensor(blocks, dtype=torch.long, device=device)[:, None] * d + torch.arange(d, device=device)[None, :]
        return idx.reshape(-1)

    def bind(self, tensors, dtype, device) -> None:
        n = self.name
        f = lambda t: tensors[f"{n}.{t}"].float()
        self.lam = float(torch.exp((f("lq1") * f("lk1")).sum()) - torch.exp((f("lq2") * f("lk2")).sum())) + self.diff
        order = self._query_order(device)
        if self.taps:
            self.conv_w = torch.cat([tensors[f"{n}.q.conv"][order], tensors[f"{n}.k.conv"], tensors[f"{n}.v.conv"]],
                                    dim=0).contiguous()
            self.conv_wt = self.conv_w.t().contiguous()
            self._no_state = torch.zeros((1, 0, self.conv_width), dtype=torch.float32, device=device)

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        w = self.proj.weight
        self.proj.use_weight(torch.cat([w[:self.q_width][self._query_order(w.device)], w[self.q_width:]], dim=0).contiguous())

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._heads_out(ctx, x, cache), residual, residual=residual)

    def mix(self, ctx, x, cache, tag: str = "mix_out"):
        o = self._heads_out(ctx, x, cache)
        return self.out.forward(ctx, o, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def _heads_out(self, ctx, x, cache):
        T, H, G, C = x.shape[0], self.n_heads, self.n_kv_heads, self.conv_width
        kv = cache.side("kv") if self.taps > 1 else cache
        es = x.element_size()
        qkv = ctx.ws.get("attn_proj", T, (C + 7) // 8 * 8, x.dtype)[:, :C]
        self.proj.forward(ctx, x, qkv)
        if self.taps:
            conv = ctx.ws.get("attn_conv", T, (C + 7) // 8 * 8, x.dtype)[:, :C]
            ops.label(self.name + ".conv", 2.0 * self.taps * T * C, 2.0 * es * T * C)
            if self.taps > 1:
                st = cache.side("conv")
                state, slots = st.state, st.slots
            else:
                state, slots = self._no_state, ctx._slots
            ops.conv_silu(qkv, self.conv_w, None, state, slots, ctx.positions, ctx.token_req, ctx.req_first_token,
                          ctx.req_first_position, conv, ctx.stream, weight_by_tap=self.conv_wt, activation=False)
            qkv = conv
        q = ctx.ws.get("attn_q32", T, 2 * H * self.key_row, torch.float32)
        ops.label(self.name + ".prepare", 2.0 * T * C, (es + 4.0) * T * C)
        ops.qkv_prepare(qkv, 0, self.q_width, self.q_width + self.k_width, 2 * H, 2 * G, self.dim, self.vdim, None, None,
                        self.eps, None, ctx.positions, ctx.token_req, kv.block_table, kv.k, kv.v, q, kv.write, ctx.status,
                        ctx.stream)
        maps = ctx.ws.get("attn_maps", T, 2 * H * self.vdim, torch.float32)
        q_rounded = None
        if (ctx.n_portion and ctx.portion_tiles is not None and "attention_prefill_tc" in self.kernel_libs
                and x.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16 and ops.PREFILL_TC):
            # the tcgen05 kernel for portions takes the queries in bfloat16
            q_rounded = ctx.ws.get("attn_q16", T, 2 * H * self.key_row, torch.bfloat16)
            ops.label(self.name + ".prepare.cast", 0.0, 6.0 * T * 2 * H * self.key_row)
            ops.join_rows(q, None, q_rounded, ctx.stream)
        if ops.recording():
            pairs, keys = visible_pairs(ctx, None, None)
            ops.label(self.name + ".maps.attention", pairs * 2 * H * (2.0 * self.dim + 2.0 * self.vdim),
                      es * keys * G * (2 * self.key_row + self.value_row) + 4.0 * T * 2 * H * (self.dim + self.vdim))
        ops.attention_wide_step(ctx, q, self.key_row, kv.k, kv.v, kv.block_table, maps, self.vdim, 2 * H, self.dim,
                                self.vdim, self.scale, q_rounded=q_rounded)
        o = ctx.ws.get("attn_out", T, H * self.vdim, x.dtype)
        ops.label(self.name + ".difference", 6.0 * T * H * self.vdim, (8.0 + es) * T * H * self.vdim)
        ops.head_difference(maps, H // G, self.vdim, self.lam, self.eps, 1.0 - self.diff, o, ctx.stream,
                            token_req=ctx.token_req)
        return o


register_part("mixer", "sink_attention", SinkAttention)
register_part("mixer", "differential_attention", DifferentialAttention)
register_part("mixer", "talking_heads_attention", TalkingHeadsAttention)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "parallel", ParallelMixer)
