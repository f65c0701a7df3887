"""Causal self-attention over the paged cache.

One fused projection gives queries, keys and values (the reference splits the
fused ``c_attn`` matrix into three at load, engine/src/gpt2.c:79-90; here it
stays one product).  Head ``h`` is the column range ``h*D .. h*D+D-1`` of q, k,
v and of the output (engine/src/attention.c:78-87).  Scores are
``(q . k) * score_scale`` over the keys at positions ``<=`` the query's
(engine/src/attention.c:24-35, engine/src/softmax.c:29-55); the softmax and
the weighted sum of values run in 32-bit.  The output projection adds its
result and bias onto the block's input (engine/src/transformer_block.c:60-62).

The keys and values of this step's tokens are first stored into the request's
pages; attention then reads the cache only, so a prompt portion and a single
decoded token take the same path.

A position encoding that acts on queries and keys (a rotation, for instance)
is a parameter of the mixer: ``position``, the description of a
``PositionEncoding`` part with ``rotate(ctx, q, k, n_heads, n_kv_heads,
head_size)``, which changes the step's queries [T, heads * head_size] and
keys [T, kv_heads * head_size] in place, each row by its ``ctx.positions``.
The projection then writes q, k and v side by side, the encoding rotates, and
the keys and values are stored into the pages by a pass of their own (the
fused projection, which scatters straight into the pages, knows no rotation).
"""

from __future__ import annotations

from .base import Mixer, build_part, register_part
from .spec import PagedKV, WeightSpec


class CausalSelfAttention(Mixer):
    graph_safe = True
    wants_attention_tiles = True      # its prompt kernel reads the step's work list of (128 queries, entry) tiles
    # (set per instance: its head count if it can also read a work list of units of 256 queries, else 0)
    attention_unit_heads = 0
    def __init__(self, prefix, width: int, n_heads: int, head_size: int, score_scale: float,
                 n_kv_heads: int | None = None, window: int | None = None,
                 qkv_name: str = "c_attn", out_name: str = "c_proj", stored_in_out: bool = True,
                 position=None):
        super().__init__(prefix)
        self.width = int(width)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads if n_kv_heads is not None else n_heads)
        self.head_size = int(head_size)
        self.attention_unit_heads = self.n_heads if self.head_size == 64 else 0
        self.score_scale = float(score_scale)
        self.window = int(window) if window else None
        self.qkv_name, self.out_name = qkv_name, out_name
        self.stored_in_out = bool(stored_in_out)
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        if self.head_size % 16 != 0 or not 16 <= self.head_size <= 256:
            raise ValueError(f"{prefix}: head size {self.head_size} is not a multiple of 16 in 16..256")
        self.position = build_part(position) if position is not None else None
        if self.position is not None:
            if not hasattr(self.position, "rotate"):
                raise ValueError(f"{prefix}: the position encoding '{position.kind}' has no rotate(ctx, q, k, ...)")
            self.graph_safe = bool(getattr(self.position, "graph_safe", False))
        self.q_width = self.n_heads * self.head_size
        self.kv_width = self.n_kv_heads * self.head_size
        self.qkv_width = self.q_width + 2 * self.kv_width

    def _matrix_shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored_in_out else (n_out, n_in)

    def weight_specs(self):
        t = self.stored_in_out
        return (self.position.weight_specs() if self.position is not None else []) + [
            WeightSpec(self.full_name(f"{self.qkv_name}.weight"), self._matrix_shape(self.width, self.qkv_width), transpose=t),
            WeightSpec(self.full_name(f"{self.qkv_name}.bias"), (self.qkv_width,), role="vector", init="bias"),
            WeightSpec(self.full_name(f"{self.out_name}.weight"), self._matrix_shape(self.q_width, self.width), transpose=t,
                       init="residual_matrix"),
            WeightSpec(self.full_name(f"{self.out_name}.bias"), (self.width,), role="vector", init="bias"),
        ]

    def cache_need(self):
        return PagedKV(self.n_kv_heads, self.head_size, self.window)

    accepts_deferred_norm = True

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        if self.position is not None:
            self.position.bind({w.name: tensors[w.name] for w in self.position.weight_specs() if w.name in tensors},
                               runtime)

    def forward(self, ctx, x, hidden, cache):
        k = ctx.kernels
        if self.position is None:
            q = k.qkv_projection(ctx, x, self.w(f"{self.qkv_name}.weight"), self.w(f"{self.qkv_name}.bias"), cache,
                                 self.q_width, self.kv_width)
        else:
            qkv = ctx.buffer("qkv", (x.shape[0], self.qkv_width), ctx.act_dtype)
            k.linear(ctx, qkv, x, self.w(f"{self.qkv_name}.weight"), self.w(f"{self.qkv_name}.bias"))
            q, keys = qkv[:, :self.q_width], qkv[:, self.q_width:self.q_width + self.kv_width]
            self.position.rotate(ctx, q, keys, self.n_heads, self.n_kv_heads, self.head_size)
            if cache.writes:
                k.kv_store(cache.k_pages, cache.v_pages, keys, qkv[:, self.q_width + self.kv_width:], ctx.positions,
                           ctx.token_item, cache.block_table, cache.page_size)
        mixed = ctx.buffer("attn_out", (q.shape[0], self.q_width), ctx.act_dtype)
        k.attention(ctx, mixed, q, cache, self.n_heads, self.n_kv_heads, self.head_size, self.score_scale,
                    self.window or 0)
        k.linear(ctx, hidden, mixed, self.w(f"{self.out_name}.weight"), self.w(f"{self.out_name}.bias"),
                 epilogue="add")


register_part("causal_self_attention", CausalSelfAttention)
