"""Arrangements: how one layer's parts are wired around the residual stream.

"pre_norm" is the reference's block (engine/src/transformer_block.c:49-71):
``r = x + mixer(norm_1(x))``, then ``out = r + feed_forward(norm_2(r))``.  The
residual stream stays 32-bit; mixers and feed-forwards add into it in place.
"""

from __future__ import annotations

from .base import Arrangement, register_arrangement


def _defer(norm, consumer) -> dict:
    if getattr(consumer, "accepts_deferred_norm", False) and getattr(norm, "can_defer", False):
        return {"defer": True}
    return {}


class PreNorm(Arrangement):
    roles = ("norm_1", "mixer", "norm_2", "feed_forward")

    def run(self, ctx, parts, hidden, cache):
        # A part that states ``accepts_deferred_norm`` may get its input norm unevaluated
        # (to fuse it into its first product); any other part gets a tensor.
        x = parts["norm_1"].forward(ctx, hidden, tag="norm_1", **_defer(parts["norm_1"], parts["mixer"]))
        parts["mixer"].forward(ctx, x, hidden, cache)
        x = parts["norm_2"].forward(ctx, hidden, tag="norm_2", **_defer(parts["norm_2"], parts["feed_forward"]))
        parts["feed_forward"].forward(ctx, x, hidden)


register_arrangement("pre_norm", PreNorm())
