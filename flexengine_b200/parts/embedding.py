"""Token embedding: the residual stream starts as the rows of a table.

x = embed_tokens.weight[ids] over the step's flattened tokens
(src/flexengine/inference/models/qwen2.py:90,94).  The stream is float32 whatever the table's dtype.
A design may scale the rows by a constant, and may start several copies of the stream at once
(``streams``: the result is then [streams, T, hidden], every copy the same).
"""
from __future__ import annotations

from .base import Embedding, register_embedding


class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, streams: int | None = None):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale, self.streams = float(scale), None if streams is None else int(streams)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, ctx):
        if self.scale == 1.0 and self.streams is None:
            return ctx.ops.embedding(ctx.token_ids, self.weight)
        return ctx.ops.embedding(ctx.token_ids, self.weight, scale=self.scale, streams=self.streams)


class HashedPairEmbedding(Embedding):
    """The token's row plus a row of a second table that is indexed by a hash of (previous token, token):
    row (previous * mul_prev + token * mul_cur) mod buckets, and row ``buckets`` (the last) for a sequence's first
    token.  The previous token of every request is kept between steps in a state group of one int32
    (``state_group`` of the plan), so that a portion that starts in mid-sequence finds it."""

    def __init__(self, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, state_group: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.state_group = int(state_group)
        self.weight = self.pairs_weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix"),
                "pairs.weight": ((self.buckets + 1, self.hidden_size), "matrix")}

    @staticmethod
    def cache_need():
        return {"kind": "state", "state_shape": (1,), "state_dtype": "int32"}

    def forward(self, ctx):
        previous = ctx.groups[self.state_group].state(0)
        return ctx.ops.embedding_hashed_pairs(ctx.token_ids, self.weight, self.pairs_weight, previous, ctx.state_slots,
                                              ctx.cu_q, ctx.q_start, ctx.token_request, self.buckets, self.mul_prev,
                                              self.mul_cur)


register_embedding("token_table", TokenEmbedding)
register_embedding("hashed_pairs", HashedPairEmbedding)
