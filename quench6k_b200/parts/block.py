"""Arrangement of the parts in a block.  "prenorm": h += mixer(norm1(h)); h += ffn(norm2(h)),
the residual stream h staying FP32 (reference: crates/engine/src/flint.rs:815-1075, :617)."""
from __future__ import annotations

from .. import ops
from .base import Block, PostNormed, ScaledSum, WeightedRows, register_block
from .norm import RMSNorm


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, h, ctx, cache, state, pending=None):
        if pending is not None and not (isinstance(pending, WeightedRows) and self.norm1.fuses_weighted_rows):
            pending.apply(h)
            pending = None
        ops.current_tag = "norm.mixer"
        xn = self.norm1.forward(h, add=pending)         # the add the block before left is made here
        delta = self.mixer.forward(xn, ctx, cache, state, h)
        ops.current_tag = "norm.ffn"
        xn = self.norm2.forward(h, add=delta)           # h += delta inside the norm when the mixer returned its result
        if self.ffn.defers_add:
            return self.ffn.forward(xn, ctx, h, defer=True)
        self.ffn.forward(xn, ctx, h)
        return None


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm on both sides of each sublayer: h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h))); a block without
    a feed-forward has the first half only.  The closing add of a sublayer is left to the norm that opens the next one
    (this block's, or the next block's first), which makes both in one pass over the row."""
    takes_extra = True

    def forward(self, h, ctx, cache, state, pending=None, extra=None):
        ops.current_tag = "norm.mixer"
        xn = self.norm1.forward(h, add=pending, extra=extra)
        y = self.mixer.forward(xn, ctx, cache, state, None)
        if y is None:
            raise TypeError(f"{type(self.mixer).__name__} adds into the stream itself; this arrangement needs its result")
        if self.ffn is None:
            return PostNormed(y, self.norm1b)
        ops.current_tag = "norm.ffn"
        xn = self.norm2.forward(h, add=PostNormed(y, self.norm1b))
        return PostNormed(self.ffn.compute(xn, ctx), self.norm2b)


@register_block("parallel")
class ParallelBlock(Block):
    """Mixer and feed-forward side by side, each behind a norm of its own, both reading the same stream:
    h += scale * (mixer(norm1(h)) + ffn(norm2(h))); a block without a feed-forward adds the mixer alone.  A block built
    without a second norm although it has a feed-forward gives both sublayers the first norm's output.  The add is left
    to the next block (or the model's last norm); with RMS norms of one eps, one kernel makes the add the block before has
    left and both norms in one pass over the row."""

    def __init__(self, norm1, mixer, norm2, ffn, scale: float = 1.0, **after):
        super().__init__(norm1, mixer, norm2, ffn, **after)
        self.scale = float(scale)

    def forward(self, h, ctx, cache, state, pending=None):
        ops.current_tag = "norm.both"
        n1, n2 = self.norm1, self.norm2
        fused = isinstance(n1, RMSNorm) and (n2 is None or (isinstance(n2, RMSNorm) and n2.eps == n1.eps))
        if fused:
            if pending is not None and not isinstance(pending, ScaledSum):
                pending.apply(h)
                pending = None
            p = pending or ScaledSum(0.0)
            w = p.weighted
            x1, x2 = ops.scaled_add_norm(h, p.a, p.b, None if w is None else (w.y, w.pair_row, w.weights), p.scale, n1.weight,
                                         n2.weight if n2 is not None else None, n1.eps, n1.rt.dtype, bias=p.bias)
        else:
            if pending is not None:
                pending.apply(h)
            x1 = n1.forward(h)
            x2 = n2.forward(h) if n2 is not None else None
        if n2 is None:
            x2 = x1                                       # one norm for both sublayers
        ctx.hold_results = self.ffn is not None           # the mixer's result waits while the feed-forward runs
        ctx.leave_bias = True                             # a mixer whose last projection has a bias may leave it to the add
        ctx.left_bias = None
        y = self.mixer.forward(x1, ctx, cache, state, None)
        ctx.hold_results = ctx.leave_bias = False
        bias = ctx.left_bias
        if y is None:
            raise TypeError(f"{type(self.mixer).__name__} adds into the stream itself; this arrangement needs its result")
        if self.ffn is None:
            return ScaledSum(self.scale, y, bias=bias)
        if hasattr(self.ffn, "compute") and not getattr(self.ffn, "defers_add", False):
            return ScaledSum(self.scale, y, self.ffn.compute(x2, ctx), bias=bias)
        if self.ffn.defers_add and getattr(self.ffn, "shared", None) is not None and hasattr(self.ffn, "compute"):
            both, rows = self.ffn.compute(x2, ctx)        # what every token shares (possibly split-K slices) and the routed rows, unsummed
            return ScaledSum(self.scale, y, both, rows, bias=bias)
        if self.ffn.defers_add:
            acc = None
            rows = self.ffn.forward(x2, ctx, None, defer=True) if getattr(self.ffn, "always_defers", False) else None
            if rows is None:
                acc = h.new_zeros(h.shape)
                rows = self.ffn.forward(x2, ctx, acc, defer=True)
            return ScaledSum(self.scale, y, acc, rows, bias=bias)
        acc = h.new_zeros(h.shape)
        self.ffn.forward(x2, ctx, acc)
        return ScaledSum(self.scale, y, acc, bias=bias)


@register_block("outnorm")
class OutNormBlock(Block):
    """A norm on each sublayer's result only: h += norm1(mixer(h)); h += norm2(ffn(h)); h += side.norm(side(h)), the
    sublayers reading the stream itself (in the operand dtype).  A block may lack the feed-forward, the side sublayer or
    both.  Each closing add is made by the kernel that also hands the stream to the next sublayer, one pass over the row;
    the block's last add is left to the block after it (or to the model's last norm)."""

    def _close(self, h, pending, dtype):
        """Makes the add that is left and returns the stream as it then stands, in the operand dtype."""
        if isinstance(pending, PostNormed) and isinstance(pending.norm, RMSNorm):
            return pending.norm.add_normed(h, pending.y, weighted=pending.weighted, out_dtype=dtype)
        if pending is not None:
            pending.apply(h)
        return ops.add_normed(h, None, None, 0.0, dtype)

    def forward(self, h, ctx, cache, state, pending=None):
        dtype = self.mixer.rt.dtype
        ops.current_tag = "stream.mixer"
        x = self._close(h, pending, dtype)
        y = self.mixer.forward(x, ctx, cache, state, None)
        if y is None:
            raise TypeError(f"{type(self.mixer).__name__} adds into the stream itself; this arrangement needs its result")
        left = PostNormed(y, self.norm1)
        if self.ffn is not None:
            ops.current_tag = "stream.ffn"
            x = self._close(h, left, dtype)
            if getattr(self.ffn, "defers_add", False):
                y, rows = self.ffn.compute(x, ctx)            # (the part every token shares or None, the routed rows unsummed)
                left = PostNormed(y, self.norm2, rows)
            else:
                left = PostNormed(self.ffn.compute(x, ctx), self.norm2)
        if self.side is not None:
            ops.current_tag = "stream.side"
            x = self._close(h, left, dtype)
            left = PostNormed(self.side.compute(x, ctx), self.side.norm)
        return left
