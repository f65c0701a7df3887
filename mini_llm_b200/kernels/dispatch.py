"""Which kernel runs an operation.

``Kernels`` is what parts call.  With ``plain_only`` (always the case for the
32-bit path) every operation runs its plain kernel.  Otherwise a fast kernel is
asked first whether it takes the sizes at hand; if it does not, the plain
kernel runs: never a wrong result, never a CPU path.
"""

from __future__ import annotations

import torch

from . import ops


class Kernels:
    def __init__(self, act_dtype: torch.dtype, plain_only: bool = False):
        self.act_dtype = act_dtype
        self.plain_only = bool(plain_only) or act_dtype == torch.float32
        self.launches = 0            # kernels launched since the counter was last reset

    # ---- operations without a fast variant --------------------------------------------------
    def embed(self, out, token_ids, positions, table, position_table=None):
        self.launches += 1
        return ops.embed(out, token_ids, positions, table, position_table)

    def add_position_rows(self, hidden, positions, table):
        self.launches += 1
        return ops.add_position_rows(hidden, positions, table)

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        self.launches += 1
        return ops.layernorm(out, x, gamma, beta, eps, rows)

    def kv_store(self, k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size):
        self.launches += 1
        return ops.kv_store(k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size)

    def sample_rows(self, out, logits, temperature=None, top_p=None, seeds=None, counters=None):
        self.launches += 1
        return ops.sample_rows(out, logits, temperature, top_p, seeds, counters)

    # ---- operations with fast variants ------------------------------------------------------
    def linear(self, out, a, w, bias=None, epilogue="store"):
        self.launches += 1
        return ops.linear_plain(out, a, w, bias, epilogue)

    def attention(self, ctx, out, q, cache, n_heads, n_kv_heads, head_size, scale, window=0):
        self.launches += 1
        return ops.attention_plain(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                   ctx.token_item, n_heads, n_kv_heads, head_size, cache.page_size, scale, window)
