"""A model as data: an embedding, a position encoding, a list of blocks, the
order in which they run, a final norm and an output head.

``ModelDescription`` is what an architecture's builder returns.  Its
``order`` is a list of ``RunEntry``: which block runs, which cache it uses and
whether it writes to it.  A block may appear twice in the order, and a block
may read the cache another block wrote (``cache`` = that block's index,
``write=False``).  ``Model`` binds loaded tensors to the parts and runs a
step: it is the only place that walks the order.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .base import MATRIX, Block, Init, Norm, ParamSpec, Part, PositionEncoding
from .linear import Linear


@dataclass(frozen=True)
class RunEntry:
    block: int                   # index into ModelDescription.blocks
    cache: Optional[int] = None  # number of the cache this run uses (None: the block's own, its index)
    write: bool = True           # whether this run appends its keys/values or state to that cache

    @property
    def cache_id(self) -> int:
        return self.block if self.cache is None else self.cache


@dataclass(frozen=True)
class Reentry:
    """A place in the run order where the stream is made anew from itself and the embedding output:
    ``x <- reentries[part].forward(ctx, x, x0, index)``.  A model that runs a span of blocks several times puts one
    before every pass and gives each pass's runs cache numbers of their own."""
    part: int                    # index into ModelDescription.reentries
    index: int = 0               # which pass this is


class TokenEmbedding(Part):
    """``h = table[token] * scale (+ position table[position])`` (mlx_lm/models/gpt2.py:132, 144)."""
    replayable = True
    kernel_libs = ("embed",)

    def __init__(self, name: str, vocab_size: int, width: int, scale: float = 1.0, init: Init = Init(),
                 weight_suffix: str = ".weight", stream_dtype: Optional[torch.dtype] = None):
        self.name, self.vocab_size, self.width, self.scale, self.init = name, vocab_size, width, scale, init
        self.weight_name = name + weight_suffix
        self.stream_dtype = stream_dtype     # dtype of the rows it writes (None: the table's); float32 for a float32 stream
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.weight_name, (self.vocab_size, self.width), MATRIX, self.init)]

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors[self.weight_name]

    def forward(self, ctx, position: Optional[PositionEncoding]):
        x = ctx.ws.get("residual", ctx.n_tokens, self.width, self.stream_dtype or self.table.dtype)
        table = position.embedding_table() if position is not None else None
        ops.label(self.name, ctx.n_tokens * self.width, (3 if table is not None else 2) * x.element_size() * ctx.n_tokens * self.width)
        freq = position.embedding_frequencies() if position is not None else None
        ops.embed_pos(ctx.tokens, ctx.positions, self.table, table, x, ctx.status, ctx.stream, scale=self.scale,
                      freq=freq)
        return x


class OutputHead(Part):
    """Logits in float32.  Tied: the embedding table is the weight and there is no bias
    (``wte.as_linear``, mlx_lm/models/gpt2.py:166-167); untied: a linear layer of its own."""
    replayable = True

    def __init__(self, vocab_size: int, width: int, tied_to: Optional[TokenEmbedding] = None,
                 name: str = "lm_head", bias: bool = False, weight_suffix: str = ".weight", init: Init = Init()):
        self.vocab_size, self.width, self.tied_to = vocab_size, width, tied_to
        self.linear = Linear(name, width, vocab_size, bias=bias and tied_to is None, weight_suffix=weight_suffix,
                             init=init)

    def children(self):
        return () if self.tied_to is not None else (self.linear,)

    def all_kernel_libs(self):
        return list(self.linear.kernel_libs)

    def bind(self, tensors, dtype, device) -> None:
        if self.tied_to is not None:
            self.linear.use_weight(self.tied_to.table)

    def forward(self, ctx, x):
        out = ctx.ws.get("logits", x.shape[0], self.vocab_size, torch.float32)
        out = self.linear.forward(ctx, x, out)
        ops.label("after the output head")
        return out


@dataclass
class ModelDescription:
    model_type: str
    width: int
    vocab_size: int
    embedding: TokenEmbedding
    position: Optional[PositionEncoding]
    blocks: List[Block]
    final_norm: Optional[Norm]
    head: OutputHead
    order: List[object] = field(default_factory=list)    # RunEntry and Reentry, in the order they run
    ignored_tensors: Sequence[str] = ()   # regular expressions of tensor names a file may hold and the model drops
    args: object = None
    reentries: List[Part] = field(default_factory=list)  # parts a Reentry of the order names
    extras: List[Part] = field(default_factory=list)     # parts that only hold tensors other parts share (a table, say)

    def __post_init__(self):
        if not self.order:
            self.order = [RunEntry(i) for i in range(len(self.blocks))]
        for e in self.order:
            if isinstance(e, Reentry):
                if not 0 <= e.part < len(self.reentries):
                    raise ValueError(f"run order names reentry {e.part} of {len(self.reentries)}")
            elif not 0 <= e.block < len(self.blocks) or e.cache_id < 0:
                raise ValueError(f"run order names block {e.block} / cache {e.cache_id} of {len(self.blocks)} blocks")
        self.cache_owner()

    def runs(self) -> List[RunEntry]:
        return [e for e in self.order if isinstance(e, RunEntry)]

    def cache_owner(self) -> Dict[int, int]:
        """``cache number -> block`` whose ``cache_spec()`` describes it: the block of the first run that writes it.
        Every cache a run uses must be written by some run, and all its users must ask for the same spec."""
        owner: Dict[int, int] = {}
        for e in self.runs():
            if e.write:
                owner.setdefault(e.cache_id, e.block)
        for e in self.runs():
            spec = self.blocks[e.block].cache_spec()
            if not spec:
                continue
            if e.cache_id not in owner:
                raise ValueError(f"cache {e.cache_id} is read by block {e.block} but no run writes it")
            if self.blocks[owner[e.cache_id]].cache_spec() != spec:
                raise ValueError(f"cache {e.cache_id}: blocks {owner[e.cache_id]} and {e.block} ask for different caches")
        return owner

    def parts(self) -> List[Part]:
        ps: List[Part] = [self.embedding]
        if self.position is not None:
            ps.append(self.position)
        ps.extend(self.extras)
        ps.extend(self.reentries)
        ps.extend(self.blocks)
        if self.final_norm is not None:
            ps.append(self.final_norm)
        ps.append(self.head)
        return ps

    def param_specs(self) -> List[ParamSpec]:
        """Every tensor the model expects, in the order the random-weights mode draws them."""
        out: List[ParamSpec] = []
        for p in self.parts():
            out.extend(p.all_param_specs())
        names = [s.name for s in out]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"two parts name the same tensor: {dup}")
        return out

    def kernel_libs(self) -> List[str]:
        libs: List[str] = []
        for p in self.parts():
            libs.extend(p.all_kernel_libs())
        return list(dict.fromkeys(libs))

    def cache_specs(self) -> Dict[object, object]:
        """Every cache the run order uses.  A block with one cache: ``cache number -> spec``; a block whose
        ``cache_spec()`` is a dictionary (several caches under names): ``(cache number, name) -> spec``."""
        out = {}
        for c, b in self.cache_owner().items():
            spec = self.blocks[b].cache_spec()
            if isinstance(spec, dict):
                out.update({(c, name): sp for name, sp in spec.items()})
            elif spec is not None:
                out[c] = spec
        return out

    @property
    def max_positions(self) -> Optional[int]:
        return self.position.max_positions if self.position is not None else None


class Model:
    """A description bound to tensors on a device in one dtype."""

    def __init__(self, description: ModelDescription, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
                 device):
        self.description = description
        self.args = description.args
        self.model_type = description.model_type
        self.dtype, self.device = dtype, torch.device(device)
        for p in description.parts():
            p.bind_all(tensors, dtype, self.device)

    @property
    def layers(self):
        return self.description.blocks

    @property
    def vocab_size(self) -> int:
        return self.description.vocab_size

    def n_parameters(self) -> int:
        n = 0
        for s in self.description.param_specs():
            c = 1
            for d in s.shape:
                c *= d
            n += c
        return n

    def run(self, ctx) -> Optional[torch.Tensor]:
        """All of this step's tokens through the blocks in run order; float32 logits
        ``[len(ctx.logit_rows), vocab]`` at the wanted rows, or None if none is wanted."""
        d = self.description
        x = x0 = d.embedding.forward(ctx, d.position)
        if d.reentries and not isinstance(d.order[0], Reentry):
            # blocks that run before the first reentry change the stream in place: they get a copy, the embedding
            # output stays as it is for the reentries
            x = ctx.ws.get("stream", ctx.n_tokens, d.width, x0.dtype)
            ops.join_rows(x0, None, x, ctx.stream)
        for entry in d.order:
            if isinstance(entry, Reentry):
                x = d.reentries[entry.part].forward(ctx, x, x0, entry.index)
            else:
                x = d.blocks[entry.block].forward(ctx, x, ctx.cache_view(entry))
        if ctx.n_logit_rows == 0:
            return None
        if d.final_norm is not None:
            h = d.final_norm.forward(ctx, x, rows=ctx.logit_rows, tag="final_normed")
        else:
            h = ctx.gather_rows(x)
        return d.head.forward(ctx, h)


class LoopInput(Part):
    """What stands before every pass of a span of blocks that runs several times:
    ``x <- W [x ; x0] + step[index]`` with ``W`` ``[width, 2 width]`` (the stream's columns first), ``x0`` the
    embedding output and one learned vector per pass.  Reads and writes a float32 stream; the product runs in the
    run's dtype with the vector as its bias."""
    replayable = True
    kernel_libs = ("elementwise",)

    def __init__(self, width: int, times: int, in_name: str = "loop.in", step_name: str = "loop.step",
                 init: Init = Init()):
        self.width, self.times, self.step_name = width, times, step_name
        self.linear = Linear(in_name, 2 * width, width, bias=False, weight_suffix="", init=init)
        self.steps: Optional[torch.Tensor] = None

    def children(self):
        return (self.linear,)

    def param_specs(self) -> List[ParamSpec]:
        from .base import VECTOR
        return [ParamSpec(self.step_name, (self.times, self.width), VECTOR, Init(0.0, 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        self.steps = tensors[self.step_name]

    def forward(self, ctx, x, x0, index: int):
        T = x.shape[0]
        both = ctx.ws.get("loop_joined", T, 2 * self.width, ctx.dtype)
        ops.label("loop.join", 0.0, (8.0 + 2 * both.element_size()) * T * self.width)
        ops.join_rows(x, x0, both, ctx.stream)
        out = ctx.ws.get("stream", T, self.width, torch.float32)
        self.linear.bias = self.steps[index]
        return self.linear.forward(ctx, both, out)
