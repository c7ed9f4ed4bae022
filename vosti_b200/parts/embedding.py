"""The embedding table: hidden rows by token id (kernels/triton_kernels/embedding.py:62-84),
optionally multiplied by a constant `scale` in float32 (Qwen3 has none; architectures that
scale their embeddings by sqrt(hidden) name it in their spec). `out_dtype` "float32" gives float32
rows whatever the table's type: the start of a float32 residual stream (in bfloat16 serving the
same kernel writes the rows' rounding beside them and the part returns both, an `ops.StreamPair`,
for arrangements whose sublayers read the rounded stream).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Embedding, StateSpec, register_part


class TableEmbedding(Embedding):
    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int):
        super().__init__(spec, hidden_size, vocab_size)
        self.scale = float(spec.get("scale", 1.0) or 1.0)
        if not self.scale == self.scale or self.scale in (float("inf"), float("-inf")):
            raise ConfigError("embedding: scale must be a finite number")
        self.out_dtype = torch.float32 if spec.get("out_dtype") == "float32" else None
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size), init="embedding")}

    def load(self, tensors, dtype):
        self.weight = tensors["weight"]

    def table(self):
        return self.weight

    def forward(self, ctx, tokens, feedback=None):
        pair = self.out_dtype == torch.float32 and ctx.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
        return ops.embedding(tokens, self.weight, ctx.status, feedback=feedback, scale=self.scale, out_dtype=self.out_dtype,
                             rounded=pair)


register_part("embedding", "table", TableEmbedding, replace=True)


class PairHashEmbedding(Embedding):
    """A token's row plus a row chosen by the token and the one before it in its sequence:

        x = table[tok] + pairs[(prev * mul_prev + tok * mul_cur) mod buckets]

    in float32 (the start of a float32 residual stream); a sequence's first token takes the pair
    table's last row, number `buckets`. The token before the first one of a step's portion is
    per-request state: one int32 per state slot, rewritten after every step.

    Parameters: buckets, mul_prev, mul_cur; `side_width` (default 0): the model also has a table
    `side` [vocab, side_width] of per-token vectors for sublayers that read the token ids again
    (parts of role "token_input"), which this part publishes in `ctx.extras["token_table"]`
    beside the step's token ids in `ctx.extras["token_ids"]`; `names`: checkpoint names of the
    tensors `pairs` and `side` where they are not `<embedding>.pairs` / `<embedding>.side`."""

    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int):
        super().__init__(spec, hidden_size, vocab_size)
        self.buckets, self.mul_prev, self.mul_cur = int(spec["buckets"]), int(spec["mul_prev"]), int(spec["mul_cur"])
        self.side_width = int(spec.get("side_width", 0) or 0)
        if self.buckets <= 0 or not 0 <= self.mul_prev < 1 << 31 or not 0 <= self.mul_cur < 1 << 31:
            raise ConfigError("pair_hash: buckets must be positive and the multipliers in [0, 2^31)")
        self.weight = self.pairs = self.side = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"weight": WeightSpec((self.vocab_size, self.hidden_size), init="embedding"),
                 "pairs": WeightSpec((self.buckets + 1, self.hidden_size), init="embedding")}
        if self.side_width:
            specs["side"] = WeightSpec((self.vocab_size, self.side_width), init="embedding")
        return specs

    def load(self, tensors, dtype):
        self.weight, self.pairs, self.side = tensors["weight"], tensors["pairs"], tensors.get("side")
        if self.weight.dtype != self.pairs.dtype:
            self.pairs = self.pairs.to(self.weight.dtype)

    def table(self):
        return self.weight

    def state_spec(self) -> StateSpec:
        return StateSpec((1,), torch.int32)

    def forward(self, ctx, tokens, feedback=None, cache=None):
        if cache is None or cache.state is None:
            raise ConfigError("pair_hash: the embedding needs its state slots (the token before a portion)")
        rows, ids = ops.pair_embedding(tokens, self.weight, self.pairs, cache.state.view(-1), ctx, buckets=self.buckets,
                                       mul_prev=self.mul_prev, mul_cur=self.mul_cur, feedback=feedback)
        ctx.extras["token_ids"] = ids
        if self.side is not None:
            ctx.extras["token_table"] = self.side
        return rows


register_part("embedding", "pair_hash", PairHashEmbedding, replace=True)
