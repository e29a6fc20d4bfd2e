"""Hooks: parts that rewrite the float32 stream right after the embedding, or the logits.  A hook that keeps something
per request offers `cache_need()` like a mixer and takes the view as a third argument of `forward`."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateNeed
from ..weights import COMPUTE, WeightSpec
from .registry import register_part


class LearnedPositions:
    """A learned vector per position, added to the stream after the embedding: x_t += table[position_t].  The table
    is stored under the hook's own name with `max_positions` rows."""
    graph_safe = True

    def __init__(self, size: int, max_positions: int):
        self.size, self.max_positions = size, max_positions
        self.table = None

    def weight_specs(self, prefix: str):
        return [WeightSpec(prefix, (self.max_positions, self.size), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.table = weights[prefix]

    def forward(self, ctx, x) -> None:
        ops.embedding(ctx.batch.positions, self.table, x, accumulate=True)


class BigramEmbedding:
    """A second embedding chosen by the token AND the one before it: x_t += table[(prev * mul_prev + cur * mul_cur)
    mod buckets]; a sequence's first token takes the row behind the buckets (the table has buckets + 1 rows).  The
    token before a step's first one is per-request state: one int32 in the request's state slot, rewritten by every
    step, so that prompts cut anywhere and decoding (also with ids that never left the device) see the same rows."""
    graph_safe = True

    def __init__(self, size: int, buckets: int, mul_prev: int, mul_cur: int):
        if buckets < 1:
            raise ValueError("a bigram table has at least one bucket")
        self.size, self.buckets, self.mul_prev, self.mul_cur = size, int(buckets), int(mul_prev), int(mul_cur)
        self.table = None

    def cache_need(self):
        return StateNeed((1,), torch.int32)

    def weight_specs(self, prefix: str):
        return [WeightSpec(prefix, (self.buckets + 1, self.size), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.table = weights[prefix]

    def forward(self, ctx, x, cache) -> None:
        ops.bigram_add(ctx.batch.tokens, self.table, cache.state, ctx.batch, x, self.mul_prev, self.mul_cur)


register_part("hook", "learned_positions", LearnedPositions)
register_part("hook", "bigram_embedding", BigramEmbedding)
