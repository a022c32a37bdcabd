"""Parts that add to the token embedding's output (registry family "embedding").

``hashed_pair``: a table indexed by a hash of the previous and the current token,

    x_t <- x_t + B[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets]        B[buckets] for a sequence's first token

with the tensor ``name`` of shape [buckets + 1, hidden].  The previous token of a portion's first token comes from the
request's state slot (one int32), which the kernel updates with the portion's last token."""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import EmbeddingExtra, WeightSpec, MATRIX, StateNeed


@register_part("embedding", "hashed_pair")
class HashedPairEmbedding(EmbeddingExtra):
    def __init__(self, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, name: str = "bigram", prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.buckets = int(hidden_size), int(buckets)
        self.mul_prev, self.mul_cur = int(mul_prev), int(mul_cur)
        if self.buckets <= 0:
            raise ValueError("buckets must be positive")
        self.name = name
        self.table = None

    def state_need(self):
        return StateNeed((1,), "int32")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.buckets + 1, self.hidden_size), MATRIX)}

    def load(self, tensors, ops, act_dtype) -> None:
        self.table = tensors[self.name]

    def forward(self, x, batch, ops, state, copies: int = 0) -> None:
        ops.pair_embed(batch, state, self.table, self.buckets, self.mul_prev, self.mul_cur, x, copies)
