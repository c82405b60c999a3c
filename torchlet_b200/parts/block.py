"""Arrangements of a layer's parts around the residual stream.

"pre_norm": h = x + mixer(norm(x)); x' = h + feed_forward(norm(h))
(v10_triton_paged_gqa/layer/transformer_block.py:37-40).  The stream ``acc`` is
float32; mixer and feed-forward add into it.

"parallel_scaled": one norm, mixer and feed-forward side by side, a residual multiplier.

"sandwich": a norm before and behind each sub-layer: x += norm_b(f(norm_a(x))).
"""
from __future__ import annotations

from .. import ops
from .base import BLOCKS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    norm_roles = ("mixer_norm", "feed_forward_norm")

    def forward(self, ctx, acc, cache) -> None:
        x = self.norms["mixer_norm"].apply(ctx, acc)
        self.mixer.forward(ctx, x, acc, cache)
        x = self.norms["feed_forward_norm"].apply(ctx, acc)
        self.feed_forward.forward(ctx, x, acc)


@BLOCKS.register("parallel_scaled")
class ParallelScaledBlock(Block):
    """h = norm(x); x' = x + m (mixer(h) + feed_forward(h)); then the layer's token input, if it
    has one, adds m * f(x', tokens).  One norm, both sub-layers read its output; ``m`` is the
    arrangement's parameter ``residual_mult`` (default 1).  The sub-layers add into a zeroed
    float32 stream of their own, so the scaled residual sum is one float32 operation."""

    norm_roles = ("shared_norm",)

    def forward(self, ctx, acc, cache) -> None:
        m = float(self.params.get("residual_mult", 1.0))
        x = self.norms["shared_norm"].apply(ctx, acc)
        delta = ctx.buffer("parallel.delta", tuple(acc.shape), acc.dtype)
        ops.fill_zero(delta)
        self.mixer.forward(ctx, x, delta, cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(ctx, x, delta)
        ctx.flush_pending()
        token_input = self.token_input
        cast = token_input.wants_cast(ctx, acc) if token_input is not None else None
        ops.scaled_add(acc, delta, m, cast)
        if token_input is not None:
            token_input.forward(ctx, acc, m, cast=cast)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """x += post(mixer(pre(x))); then, if the layer has a feed-forward, x += post'(ff(pre'(x))).
    Each sub-layer adds its output into a zeroed float32 stream of its own, the norm behind it
    reads that stream and adds the normed rows into the residual stream (``Norm.add_normed``), so
    the sub-layer's output, its norm and the residual sum are all float32.  That norm's kernel also
    leaves the side stream zeroed again, so it is cleared by a kernel of its own once a step only."""

    norm_roles = ("mixer_norm", "mixer_post_norm")

    def __init__(self, mixer, feed_forward, norms, params=None, token_input=None):
        super().__init__(mixer, feed_forward, norms, params, token_input)
        if feed_forward is not None:
            missing = [role for role in ("feed_forward_norm", "feed_forward_post_norm") if role not in norms]
            if missing:
                raise ValueError(f"block arrangement {self.kind!r} with a feed-forward needs norms for the roles {missing}")

    def forward(self, ctx, acc, cache) -> None:
        side = ctx.buffer("sandwich.side", tuple(acc.shape), acc.dtype)
        x = self.norms["mixer_norm"].apply(ctx, acc)
        if ctx.plans.get("sandwich.side.clean") != side.data_ptr():  # the first sandwich block of the step
            ops.fill_zero(side)
            ctx.plans["sandwich.side.clean"] = side.data_ptr()
        self.mixer.forward(ctx, x, side, cache)
        self.norms["mixer_post_norm"].add_normed(ctx, side, acc, clear=True)
        if self.feed_forward is not None:
            x = self.norms["feed_forward_norm"].apply(ctx, acc)
            self.feed_forward.forward(ctx, x, side)
            self.norms["feed_forward_post_norm"].add_normed(ctx, side, acc, clear=True)
