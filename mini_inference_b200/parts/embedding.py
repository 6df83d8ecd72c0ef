"""Embedding parts: how token ids become the first rows of the residual stream when that takes more than a
lookup in the embedding table.  The model hands its embedding table in; a part owns whatever further tables it adds.

hashed_bigram   x_t = table[token_t] + pairs[(prev_t * mul_prev + token_t * mul_cur) mod buckets], prev_t being the token
                before token_t in its sequence; a sequence's first token takes the pair table's last row (row `buckets`).
                The previous token of a request is state: one int32 per slot, so that a prompt may be cut anywhere and a
                decoded token finds its predecessor on the device.  The stream starts in float32."""
from __future__ import annotations

from .base import Part, StateNeed, WeightSpec, register_embedding


@register_embedding("hashed_bigram")
class HashedBigramEmbedding(Part):
    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.buckets = int(g("hidden_size")), int(g("buckets"))
        self.mul_prev, self.mul_cur = int(g("mul_prev")), int(g("mul_cur"))
        if self.buckets < 1:
            raise ValueError("hashed_bigram needs at least one bucket")
        self.pairs = None

    def weight_specs(self):
        return [WeightSpec("pairs", (self.buckets + 1, self.hidden))]

    def cache_need(self):
        return StateNeed((1,), "int32")

    def load(self, tensors, dtype, device):
        self.pairs = tensors["pairs"]

    def forward(self, ids, table, ctx, cache):
        return ctx.ops.embed_bigram_stream(ids, table, self.pairs, self.buckets, self.mul_prev, self.mul_cur, cache.state, ctx.batch)
