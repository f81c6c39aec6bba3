"""Pre-norm block: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/llama.py:66-89).  The sums are carried as the stream's pending branch and folded in
by the next norm.  A layer without a feed-forward is the first half only.

``parallel_norms``: both branches read the same x (see ``ParallelNormsBlock``)."""

from __future__ import annotations

from ..kernels import ops
from .base import Block, register_block
from .context import CacheBinding, ResidualStream, StepContext


class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following=None) -> None:
        h = _normed(self.mixer_norm, stream, ctx)
        if self.feed_forward is None:
            ahead = None
            if following is not None:
                ahead = _ahead(self.mixer, following[0], following[1], stream, ctx)
        else:
            ahead = _ahead(self.mixer, self.feed_forward_norm, self.feed_forward, stream, ctx)
        if ahead is None:
            stream.pending = self.mixer.forward(h, ctx, cache)
        else:
            self.mixer.forward(h, ctx, cache, ahead=ahead)
            stream.ahead = ahead
        if self.feed_forward is None:
            return
        h = _normed(self.feed_forward_norm, stream, ctx)
        ahead = None
        if following is not None:
            ahead = _ahead(self.feed_forward, following[0], following[1], stream, ctx)
        if ahead is None:
            stream.pending = self.feed_forward.forward(h, ctx)
        else:
            self.feed_forward.forward(h, ctx, ahead=ahead)
            stream.ahead = ahead


def _normed(norm, stream: ResidualStream, ctx: StepContext):
    """The norm's output, from the product before it if that did the work."""
    ahead, stream.ahead = stream.ahead, None
    if ahead is None:
        return norm.forward(stream, ctx)
    if ahead.norm is not norm:
        raise RuntimeError("the stream holds another norm's work than the one that runs next")
    return ahead.result()


def _ahead(producer, norm, consumer, stream: ResidualStream, ctx: StepContext):
    """Buffers for ``producer``'s last product to do ``norm``'s work, if producer, norm and
    ``consumer`` (which must take rows without their factors) all can for this step."""
    n = stream.resid.shape[0]
    abilities = (getattr(producer, "ahead_parts", None), getattr(consumer, "takes_unscaled", None))
    if None in abilities:
        return None
    count = abilities[0](n)
    if not count or not abilities[1](n):
        return None
    return norm.ahead(stream, ctx, count)


register_block("prenorm", PreNormBlock)


class ParallelNormsBlock(Block):
    """Two branches of the same input, each behind a norm of its own:
    x += mixer(norm1(x)) + feed_forward(norm2(x)), the three terms summed in float32; then the
    layer's side input, if it has one, reads the new x and adds to it.  A layer without a
    feed-forward is x += mixer(norm1(x))."""

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following=None) -> None:
        if stream.ahead is not None:
            raise RuntimeError("a block of parallel branches runs its norms itself")
        h = self.mixer_norm.forward(stream, ctx)            # also folds what was pending
        h2 = None
        if self.feed_forward is not None:
            h2 = self.feed_forward_norm.forward(stream, ctx, out_name="norm.out.second")
        a = self.mixer.forward(h, ctx, cache)
        b = self.feed_forward.forward(h2, ctx) if self.feed_forward is not None else None
        if self.side_input is None:
            ops.residual_add(stream.resid, a, b)
            return
        rows = ctx.buffer("block.rows", tuple(stream.resid.shape))
        ops.residual_add(stream.resid, a, b, rows=rows)
        self.side_input.forward(stream, rows, ctx)


register_block("parallel_norms", ParallelNormsBlock)
