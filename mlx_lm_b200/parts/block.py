"""Arrangements of parts in a layer.  ``PreNormBlock``:
``h = x + mixer(norm_1(x)); out = h + feed_forward(norm_2(h))``
(mlx_lm/models/gpt2.py:104-108).  The residual stream is updated in place by
the epilogues of the mixer's and the feed-forward's last products."""

from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops
from .base import Block, FeedForward, Mixer, Norm, register_part

# In bfloat16 a block lets its mixer and its feed-forward fold the norm before them into their first linear
# layer (parts/linear.py, ``Linear.fold_norm``): steps of few rows then run no norm kernels inside the blocks.
# MLXB_FOLD_NORMS=0 (or setting this to False before a model is loaded) keeps every norm a kernel of its own.
FOLD_NORMS = os.environ.get("MLXB_FOLD_NORMS", "1") != "0"


class PreNormBlock(Block):
    replayable = True
    kernel_libs = ("gemm_smallm_fold", "norm")     # what folding a norm into a linear layer launches from
    def __init__(self, norm_1: Norm, mixer: Mixer, norm_2: Norm, feed_forward: FeedForward):
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self._defer_1 = self._defer_2 = False

    def children(self):
        return (self.norm_1, self.mixer, self.norm_2, self.feed_forward)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        fold = FOLD_NORMS and dtype == torch.bfloat16
        self._defer_1 = fold and self.mixer.fold_input_norm(self.norm_1)
        self._defer_2 = fold and self.feed_forward.fold_input_norm(self.norm_2)

    def forward(self, ctx, x, cache):
        n1 = self.norm_1.deferred(ctx, x) if self._defer_1 else self.norm_1.forward(ctx, x)
        h = self.mixer.forward(ctx, n1, x, cache)
        n2 = self.norm_2.deferred(ctx, h) if self._defer_2 else self.norm_2.forward(ctx, h)
        return self.feed_forward.forward(ctx, n2, h)


class StreamBlock(Block):
    """A pre-norm block over a float32 residual stream: ``x += mixer(norm_1(x))``, then, if the layer has a
    feed-forward, ``x += feed_forward(norm_2(x))``, then any number of further branches, each of which reads the
    stream and adds to it (``branch.forward(ctx, x) -> x``).  Norms give the run's dtype to the products; the sums
    stay float32 whatever the run's dtype is."""
    replayable = True

    def __init__(self, norm_1: Norm, mixer: Mixer, norm_2: Optional[Norm] = None,
                 feed_forward: Optional[FeedForward] = None, branches=()):
        if (norm_2 is None) != (feed_forward is None):
            raise ValueError("a feed-forward and the norm before it come together")
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.branches = tuple(branches)

    def children(self):
        return tuple(p for p in (self.norm_1, self.mixer, self.norm_2, self.feed_forward) if p is not None) + self.branches

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        x = self.mixer.forward(ctx, self.norm_1.forward(ctx, x), x, cache)
        if self.feed_forward is not None:
            x = self.feed_forward.forward(ctx, self.norm_2.forward(ctx, x), x)
        for b in self.branches:
            x = b.forward(ctx, x)
        return x


class ParallelBlock(Block):
    """A block over a float32 residual stream whose two sublayers read the same normed input:
    ``h = norm_1(x); x += mixer(h) + feed_forward(h)``.  There is one norm; the feed-forward is optional.  Each
    sublayer adds its result to the stream itself (the mixer in its last product's epilogue)."""
    replayable = True

    def __init__(self, norm_1: Norm, mixer: Mixer, feed_forward: Optional[FeedForward] = None):
        self.norm_1, self.mixer, self.feed_forward = norm_1, mixer, feed_forward

    def children(self):
        return tuple(p for p in (self.norm_1, self.mixer, self.feed_forward) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        h = self.norm_1.forward(ctx, x)
        x = self.mixer.forward(ctx, h, x, cache)
        if self.feed_forward is not None:
            x = self.feed_forward.forward(ctx, h, x)
        return x


class SandwichBlock(Block):
    """A block over a float32 residual stream with a norm before AND after each sublayer:
    ``x += post_1(mixer(norm_1(x)))``, then, if the layer has a feed-forward, ``x += post_2(feed_forward(norm_2(x)))``.

    The sublayers leave their results in float32 (``mixer.mix(ctx, x, cache) -> [T, width]``,
    ``feed_forward.branch(ctx, x) -> ([T * terms, width], terms)``: a feed-forward of experts hands over one row per
    (token, chosen expert), summed in the update).  The post-norms are elementwise (``Norm.stream_args()``), so one
    kernel does the sum over terms, the post-norm, the add to the stream and the norm that reads the stream next:
    ``norm_2`` of this block, or ``norm_1`` of the block named by ``feeds`` (the one that runs next), whose input
    then waits in ``ctx.carried``.  Norms in front that are not elementwise run as kernels of their own."""
    replayable = True
    kernel_libs = ("dyt",)

    def __init__(self, norm_1: Norm, mixer: Mixer, post_1: Norm, norm_2: Optional[Norm] = None,
                 feed_forward: Optional[FeedForward] = None, post_2: Optional[Norm] = None,
                 feeds: Optional["SandwichBlock"] = None):
        if not (norm_2 is None) == (feed_forward is None) == (post_2 is None):
            raise ValueError("a feed-forward comes with the norm before it and the norm after it")
        self.norm_1, self.mixer, self.post_1 = norm_1, mixer, post_1
        self.norm_2, self.feed_forward, self.post_2 = norm_2, feed_forward, post_2
        self.feeds = feeds

    def children(self):
        return tuple(p for p in (self.norm_1, self.mixer, self.post_1, self.norm_2, self.feed_forward, self.post_2)
                     if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @staticmethod
    def _fusable(norm: Optional[Norm]) -> bool:
        return norm is not None and hasattr(norm, "stream_args") and getattr(norm, "out_scale", 1.0) == 1.0

    def _update(self, ctx, x, branch, terms: int, post: Norm, nxt: Optional[Norm], tag: str, name: str):
        T, D = x.shape
        out = None
        if self._fusable(nxt):
            out = ctx.ws.get(tag, T, D, ctx.dtype)
        ops.label(name, (12.0 + terms) * T * D, (8.0 + 4.0 * terms + (out.element_size() if out is not None else 0)) * T * D)
        ops.dyt_residual(x, branch, ctx.stream, post=post.stream_args(), nxt=nxt.stream_args() if out is not None else None,
                         next_out=out, terms=terms, token_req=ctx.token_req)
        return out

    def forward(self, ctx, x, cache):
        carried = getattr(ctx, "carried", None)
        ctx.carried = None
        if carried is not None and carried[0] is self.norm_1:
            n1 = carried[1]
        else:
            n1 = self.norm_1.forward(ctx, x)
        y = self.mixer.mix(ctx, n1, cache)
        if self.feed_forward is None:
            nxt = self.feeds.norm_1 if self.feeds is not None else None
            out = self._update(ctx, x, y, 1, self.post_1, nxt, "normed", self.post_1.name)
            if out is not None:
                ctx.carried = (nxt, out)
            return x
        n2 = self._update(ctx, x, y, 1, self.post_1, self.norm_2, "normed_2", self.post_1.name)
        if n2 is None:
            n2 = self.norm_2.forward(ctx, x, tag="normed_2")
        yb, terms = self.feed_forward.branch(ctx, n2)
        nxt = self.feeds.norm_1 if self.feeds is not None else None
        out = self._update(ctx, x, yb, terms, self.post_2, nxt, "normed", self.post_2.name)
        if out is not None:
            ctx.carried = (nxt, out)
        return x


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "stream", StreamBlock)
