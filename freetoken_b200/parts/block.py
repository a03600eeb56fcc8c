"""Arrangements of a mixer and a feed-forward around the residual stream.

``prenorm`` is the reference's decoder layer
(python/freetoken/models/minimax_m2/model.py:27-37): the layer receives the
previous branch output ``delta`` and the float32 ``residual``; each norm first
adds the pending branch output into the residual, then normalises::

    h = norm1(delta, residual)      # residual += delta
    a = mixer(h)
    h = norm2(a, residual)          # residual += a
    return feed_forward(h)          # the next norm adds it

``parallel`` has ONE norm whose output both sublayers read; the layer adds the
sum of their outputs::

    h = norm(delta, residual)       # residual += delta
    return [mixer(h), feed_forward(h)]   # two partial rows per token

The two outputs leave the block as ``[T, 2, H]``; the next norm adds them to each
other and then to the residual in float32 (``x + (mixer + feed_forward)``).  A
parallel layer may have no feed-forward; then it returns the mixer's rows alone.

``sandwich`` norms every sublayer's output as well as its input and scales it before it
joins the residual stream::

    h = norm_in(delta, residual)                  # residual += delta
    residual += mult * norm_out(mixer(h))
    residual += mult * norm_out'(feed_forward(norm_in'(residual)))

Both sums happen in float32 inside the norm kernel that computes the output norm; the
output norm of the mixer and the input norm of the feed-forward are one launch.  The
block leaves nothing pending (it returns ``None``).

``hyper`` is a pre-norm block over several residual streams (hyper-connections): each of its
norms (:class:`~.norm.HyperNorm`) forms its sublayer's input from all streams and owns the weights
by which the sublayer's output joins them; the output travels on as a pending branch that the
next such norm folds in::

    h = norm1(pending, streams)            # the pending branch joins the streams; u = sum_s in1[s] x_s
    pending = (mixer(h), mix1, out1)
    h = norm2(pending, streams)
    return (feed_forward(h), mix2, out2)   # the next layer's first norm (or the last norm) adds it
"""

from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    NORM_NAMES = ("mixer", "feed_forward")
    HAS_FEED_FORWARD = True

    def forward(self, ctx, delta, residual, cache):
        h = self.mixer_norm.forward(ctx, delta, residual)
        a = self.mixer.forward(ctx, h, cache)
        h = self.feed_forward_norm.forward(ctx, a, residual)
        return self.feed_forward.forward(ctx, h)


@register_block("parallel")
class ParallelBlock(Block):
    NORM_NAMES = ("mixer",)
    HAS_FEED_FORWARD = True          # or none: see check_parts

    @classmethod
    def check_parts(cls, prefix, norm_names, has_feed_forward) -> None:
        if sorted(norm_names) != sorted(cls.NORM_NAMES):
            raise ValueError(f"layer '{prefix}': a parallel block has the one norm {list(cls.NORM_NAMES)}, "
                             f"the layer lists {sorted(norm_names)}")

    def forward(self, ctx, delta, residual, cache):
        h = self.mixer_norm.forward(ctx, delta, residual)
        if self.feed_forward is None:
            return self.mixer.forward(ctx, h, cache)
        T, H = h.shape
        pair = ctx.workspace.get("block.pair", (T, 2, H), ctx.dtype)
        if self.mixer.writes_into_out:
            self.mixer.forward(ctx, h, cache, out=pair[:, 0])
        else:
            pair[:, 0].copy_(self.mixer.forward(ctx, h, cache))
        if self.feed_forward.writes_into_out:
            self.feed_forward.forward(ctx, h, out=pair[:, 1])
        else:
            pair[:, 1].copy_(self.feed_forward.forward(ctx, h))
        return pair


@register_block("sandwich")
class SandwichBlock(Block):
    """params: ``residual_mult`` (default 1): the factor on every normed sublayer output."""

    NORM_NAMES = ("mixer", "mixer_out", "feed_forward", "feed_forward_out")
    HAS_FEED_FORWARD = True          # or none: then only the mixer's two norms

    @classmethod
    def check_parts(cls, prefix, norm_names, has_feed_forward) -> None:
        want = cls.NORM_NAMES if has_feed_forward else cls.NORM_NAMES[:2]
        if sorted(norm_names) != sorted(want):
            raise ValueError(f"layer '{prefix}': a sandwich block {'with' if has_feed_forward else 'without'} "
                             f"feed-forward has the norms {list(want)}, the layer lists {sorted(norm_names)}")

    def __init__(self, spec, prefix, mixer, feed_forward, norms):
        super().__init__(spec, prefix, mixer, feed_forward, norms)
        self.mult = float(spec.get("residual_mult", 1.0))

    def forward(self, ctx, delta, residual, cache):
        h = self.norms["mixer"].forward(ctx, delta, residual)
        a = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            self.norms["mixer_out"].add_normed(ctx, a, residual, self.mult)
            return None
        h = self.norms["mixer_out"].add_normed(ctx, a, residual, self.mult, then=self.norms["feed_forward"])
        f = self.feed_forward.forward(ctx, h)
        self.norms["feed_forward_out"].add_normed(ctx, f, residual, self.mult)
        return None


@register_block("hyper")
class HyperBlock(Block):
    NORM_NAMES = ("mixer", "feed_forward")
    HAS_FEED_FORWARD = True          # or none: then only the mixer's norm

    @classmethod
    def check_parts(cls, prefix, norm_names, has_feed_forward) -> None:
        want = cls.NORM_NAMES if has_feed_forward else cls.NORM_NAMES[:1]
        if sorted(norm_names) != sorted(want):
            raise ValueError(f"layer '{prefix}': a hyper block {'with' if has_feed_forward else 'without'} "
                             f"feed-forward has the norms {list(want)}, the layer lists {sorted(norm_names)}")

    def forward(self, ctx, delta, residual, cache):
        first = self.norms["mixer"]
        h = first.forward(ctx, delta, residual)
        pending = first.pending(self.mixer.forward(ctx, h, cache))
        if self.feed_forward is None:
            return pending
        second = self.norms["feed_forward"]
        h = second.forward(ctx, pending, residual)
        return second.pending(self.feed_forward.forward(ctx, h))
