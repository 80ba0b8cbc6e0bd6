"""The arrangement of a layer: norm -> mixer -> residual, norm -> feed-forward -> residual
(the reference's two-norm pre-norm block, src/minimax.rs:261-284).  Each residual sum is
left to the norm that follows it, which adds in float32 while it reads the stream.
A second arrangement, ``output_norm``, has the norm behind the sublayer instead of in front of it; a third,
``parallel_pre_norm``, runs the two sublayers side by side on the same x; a fourth, ``sandwich_norm``, has a norm on
both sides of each sublayer."""
from __future__ import annotations

import torch

from .base import Block, NormedUpdate, UpdateSum, as_tensor, register_part
from .norm import LayerNorm


class PreNormBlock(Block):
    def forward(self, ctx, x, pending, line, writes_cache):
        if not self.mixer_norm.accepts_deferred:
            pending = as_tensor(ctx, pending)
        act, _ = self.mixer_norm.forward(ctx, x, delta=pending)
        update = self.mixer.forward(ctx, act, line, writes_cache)
        if self.feed_forward is None:                  # a layer without feed-forward: the next norm adds the mixer's update
            return x, update
        if not self.feed_forward_norm.accepts_deferred:
            update = as_tensor(ctx, update)
        act2, act2_32 = self.feed_forward_norm.forward(ctx, x, delta=update,
                                                       want32=self.feed_forward.wants_float32_input)
        return x, self.feed_forward.forward_deferred(ctx, act2, act2_32)


class OutputNormBlock(Block):
    """The norm on the sublayer's output only: x <- x + norm1(mixer(x)), then, if the layer has a feed-forward,
    x <- x + norm2(feed_forward(x)).  The sublayers read x itself, so besides the float32 stream its copy in the
    model dtype goes from sublayer to sublayer: the norm that adds to the stream writes it (``Norm.add_normed``),
    an embedding with ``typed_copy`` writes the first one."""

    def stream_copy(self, ctx, x, pending):
        if pending is not None:                            # a block before this one left its update to the next norm
            from ..csrc import ops
            ops.add_rows(x, as_tensor(ctx, pending))
            ctx.stream_copy_rows = -1
        if x.dtype == self.mixer.dtype:
            return x
        act = ctx.buffer(LayerNorm.STREAM_COPY, tuple(x.shape), self.mixer.dtype)
        if getattr(ctx, "stream_copy_rows", -1) != x.shape[0]:
            act.copy_(x)                                   # nobody wrote the copy of this step's stream yet
        return act

    def forward(self, ctx, x, pending, line, writes_cache):
        act = self.stream_copy(ctx, x, pending)
        update = as_tensor(ctx, self.mixer.forward(ctx, act, line, writes_cache))
        act = self.mixer_norm.add_normed(ctx, update, x)
        if self.feed_forward is not None:
            act32 = x if self.feed_forward.wants_float32_input else None
            update = as_tensor(ctx, self.feed_forward.forward_deferred(ctx, act, act32))
            self.feed_forward_norm.add_normed(ctx, update, x)
        ctx.stream_copy_rows = x.shape[0]
        return x, None


class ParallelPreNormBlock(Block):
    """Both sublayers side by side: x <- x + mixer(norm1(x)) + feed_forward(norm2(x)), the two norms reading the same
    x.  Their outputs are left unsummed (``UpdateSum``) for the norm that reads the stream next.  Two norms of a kind
    that has ``forward_pair`` run as one kernel."""

    def forward(self, ctx, x, pending, line, writes_cache):
        ff, norm1, norm2 = self.feed_forward, self.mixer_norm, self.feed_forward_norm
        want32 = ff is not None and ff.wants_float32_input
        if ff is not None and hasattr(norm1, "forward_pair") and type(norm1) is type(norm2):
            act1, act2, act2_32 = norm1.forward_pair(ctx, x, norm2, delta=pending, want32=want32)
            update = self.mixer.forward(ctx, act1, line, writes_cache)
        else:
            if not norm1.accepts_deferred:
                pending = as_tensor(ctx, pending)
            act1, _ = norm1.forward(ctx, x, delta=pending)
            update = self.mixer.forward(ctx, act1, line, writes_cache)       # before the second norm takes the buffer
            if ff is not None:
                act2, act2_32 = norm2.forward(ctx, x, want32=want32)
        if ff is None:
            return x, update
        return x, UpdateSum([as_tensor(ctx, update), ff.forward_deferred(ctx, act2, act2_32)])


class SandwichNormBlock(Block):
    """A norm in front of and behind each sublayer: x <- x + norm1b(mixer(norm1(x))), then, if the layer has a
    feed-forward, x <- x + norm2b(feed_forward(norm2(x))).  A sublayer's output is left with its norm
    (``NormedUpdate``) for the norm that reads the stream next, which norms the output, adds it and norms the sum in
    one pass."""

    def forward(self, ctx, x, pending, line, writes_cache):
        if self.mixer_out_norm is None or (self.feed_forward is not None and self.feed_forward_out_norm is None):
            raise ValueError("a block with norms on both sides of its sublayers was given no norm for a sublayer's output")
        act, _ = self.mixer_norm.forward(ctx, x, delta=pending)
        pending = NormedUpdate(self.mixer.forward(ctx, act, line, writes_cache), self.mixer_out_norm)
        if self.feed_forward is None:
            return x, pending
        act2, act2_32 = self.feed_forward_norm.forward(ctx, x, delta=pending, want32=self.feed_forward.wants_float32_input)
        return x, NormedUpdate(self.feed_forward.forward_deferred(ctx, act2, act2_32), self.feed_forward_out_norm)


register_part("block", "sandwich_norm", SandwichNormBlock, replace=True)
register_part("block", "parallel_pre_norm", ParallelPreNormBlock, replace=True)
register_part("block", "pre_norm", PreNormBlock, replace=True)
register_part("block", "output_norm", OutputNormBlock, replace=True)
