"""Dense feed-forward: ``act(x W_up + b_up) W_down + b_down``, added onto the
residual stream (engine/src/transformer_block.c:64-71).  The activation is a
parameter: the tanh form of gelu (engine/include/gelu_math.h:6-11) or the erf
form (engine/src/gelu.c:5-9)."""

from __future__ import annotations

from .base import FeedForward, register_part
from .spec import WeightSpec

ACTIVATION_EPILOGUES = ("gelu_tanh", "gelu_erf")


class DenseMlp(FeedForward):
    graph_safe = True
    def __init__(self, prefix, width: int, inner: int, activation: str,
                 up_name: str = "c_fc", down_name: str = "c_proj", stored_in_out: bool = True):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)
        if activation not in ACTIVATION_EPILOGUES:
            raise ValueError(f"{prefix}: unknown activation '{activation}' (known: {', '.join(ACTIVATION_EPILOGUES)})")
        self.activation = activation
        self.up_name, self.down_name = up_name, down_name
        self.stored_in_out = bool(stored_in_out)

    def _matrix_shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored_in_out else (n_out, n_in)

    def weight_specs(self):
        t = self.stored_in_out
        return [
            WeightSpec(self.full_name(f"{self.up_name}.weight"), self._matrix_shape(self.width, self.inner), transpose=t),
            WeightSpec(self.full_name(f"{self.up_name}.bias"), (self.inner,), role="vector", init="bias"),
            WeightSpec(self.full_name(f"{self.down_name}.weight"), self._matrix_shape(self.inner, self.width), transpose=t,
                       init="residual_matrix"),
            WeightSpec(self.full_name(f"{self.down_name}.bias"), (self.width,), role="vector", init="bias"),
        ]

    accepts_deferred_norm = True

    def forward(self, ctx, x, hidden):
        up = ctx.buffer("mlp_up", (x.shape[0], self.inner), ctx.act_dtype)
        ctx.kernels.linear(ctx, up, x, self.w(f"{self.up_name}.weight"), self.w(f"{self.up_name}.bias"),
                           epilogue=self.activation)
        ctx.kernels.linear(ctx, hidden, up, self.w(f"{self.down_name}.weight"), self.w(f"{self.down_name}.bias"),
                           epilogue="add")


register_part("dense_mlp", DenseMlp)
