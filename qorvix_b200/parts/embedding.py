"""Embeddings that are more than one table.  A plain table needs no part (the model gathers its rows);
an embedding part has `forward(out, ctx, cache)` filling the float32 residual stream and may keep a
small state per request (`cache_spec()`), which the cache manager zeroes at admission."""
from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec
from ..csrc import ops
from .registry import register_part


class BigramEmbedding:
    """Token row plus the row of a hashed (previous token, token) pair.  The previous token of a
    segment's first token is the request's state: one int32 per request slot."""

    def __init__(self, spec, source, rt):
        self.spec = spec
        self.table = source.get(spec.table)
        self.pair = source.get(spec.pair_table)
        if self.pair.dtype != self.table.dtype:
            self.pair = self.pair.to(self.table.dtype)

    @property
    def weight(self) -> torch.Tensor:
        return self.table

    def cache_spec(self):
        return FixedStateSpec((1,), "int32")

    def forward(self, out, ctx, cache) -> None:
        s = self.spec
        ops.embed_pair(out, self.table, self.pair, ctx.token_ids, ctx, cache.tensor.reshape(-1), s.buckets, s.mul_prev, s.mul_cur)


register_part("embedding", "bigram_embedding", BigramEmbedding)
