"""Token embedding, learned absolute positions, and the output head.

``hidden[t] = wte[id_t] + wpe[pos_t]`` with ``pos_t`` the token's absolute
position in its request (engine/src/embedding.c:9-15; with an offset for
cached tokens, engine/src/embedding.cu:21-26,100-103).  The head multiplies
the normed rows whose logits are wanted with the token table itself, without
bias (engine/src/gpt2.c:245-256); the reference keeps a transposed copy of
the table for this (engine/src/gpt2_gpu.cu:32-48), here the one [vocab, width]
table serves the gather and the product.
"""

from __future__ import annotations

import torch

from .base import Embedding, Head, PositionEncoding, register_part
from .spec import WeightSpec


class TokenEmbedding(Embedding):
    graph_safe = True
    def __init__(self, prefix, vocab_size: int, width: int, name: str = "wte.weight"):
        super().__init__(prefix)
        self.vocab_size, self.width, self.name = int(vocab_size), int(width), name

    def weight_specs(self):
        return [WeightSpec(self.full_name(self.name), (self.vocab_size, self.width), role="table", init="table")]

    def forward(self, ctx, position=None):
        hidden = ctx.buffer("hidden", (ctx.n_tokens, self.width), torch.float32)
        table = position.additive_table() if position is not None else None
        ctx.kernels.embed(hidden, ctx.token_ids, ctx.positions, self.w(self.name), table)
        if position is not None and table is None:
            position.add_to_hidden(ctx, hidden)
        return hidden


class LearnedPositions(PositionEncoding):
    """A table row per absolute position, added to the embedded token."""
    graph_safe = True

    def __init__(self, prefix, max_positions: int, width: int, name: str = "wpe.weight"):
        super().__init__(prefix)
        self.max_positions, self.width, self.name = int(max_positions), int(width), name

    def weight_specs(self):
        return [WeightSpec(self.full_name(self.name), (self.max_positions, self.width), role="table", init="table")]

    def additive_table(self):
        return self.w(self.name)

    def add_to_hidden(self, ctx, hidden):
        ctx.kernels.add_position_rows(hidden, ctx.positions, self.w(self.name))


class LinearHead(Head):
    """logits = x W^T, W [vocab, width].  ``weight_name`` may be the token
    table's name (tied head): the loader then shares the one tensor."""
    graph_safe = True

    def __init__(self, prefix, vocab_size: int, width: int, weight_name: str = "lm_head.weight"):
        super().__init__(prefix)
        self.vocab_size, self.width, self.weight_name = int(vocab_size), int(width), weight_name

    def weight_specs(self):
        return [WeightSpec(self.full_name(self.weight_name), (self.vocab_size, self.width), role="table", init="table")]

    accepts_deferred_norm = True

    def forward(self, ctx, x):
        logits = ctx.buffer("logits", (x.shape[0], self.vocab_size), torch.float32)
        ctx.kernels.linear(ctx, logits, x, self.w(self.weight_name), None)
        return logits


register_part("token_embedding", TokenEmbedding)
register_part("learned_positions", LearnedPositions)
register_part("linear_head", LinearHead)
