"""Layer norm: mean, biased variance of the centred values, then
``(x - mean) / sqrt(var + eps) * gain + shift`` (engine/src/layernorm.c:12-33).
Statistics are 32-bit; the output has the engine's element type."""

from __future__ import annotations

from ..kernels.dispatch import DeferredNorm
from .base import Norm, register_part
from .spec import WeightSpec


class LayerNorm(Norm):
    graph_safe = True
    can_defer = True

    def __init__(self, prefix, width: int, eps: float):
        super().__init__(prefix)
        self.width = int(width)
        self.eps = float(eps)

    def weight_specs(self):
        return [
            WeightSpec(self.full_name("weight"), (self.width,), role="vector", init="gain"),
            WeightSpec(self.full_name("bias"), (self.width,), role="vector", init="shift"),
        ]

    def forward(self, ctx, x, rows=None, tag="norm", defer=False):
        if defer:
            gamma, beta = self.w("weight"), self.w("bias")
            return DeferredNorm("layer_norm", x, rows, tag,
                                lambda c, out: c.kernels.layernorm(out, x, gamma, beta, self.eps, rows),
                                gamma=gamma, beta=beta, eps=self.eps)
        n_rows = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(tag, (n_rows, self.width), ctx.act_dtype)
        ctx.kernels.layernorm(out, x, self.w("weight"), self.w("bias"), self.eps, rows)
        return out


register_part("layer_norm", LayerNorm)
