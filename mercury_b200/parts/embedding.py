"""Token embedding and the output head.

Embedding: a row lookup without scaling (mercury/model/qwen2.py:100, :109), written into
the float32 residual stream. Head: hidden times the embedding table when tied, else times
its own matrix, no bias (mercury/model/qwen2.py:128-130, :145-150); logits are float32.
"""

from __future__ import annotations

from .base import Part, TensorSpec


class TokenEmbedding(Part):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight_name = weight_name
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, setup):
        self.table = setup.place(tensors[self.weight_name])

    def forward(self, token_ids, ctx):
        h = ctx.buffer("residual", token_ids.shape[0], self.hidden_size, dtype="float32")
        ctx.ops.embed(token_ids, self.table, h)
        return h


class OutputHead(Part):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str | None):
        """`weight_name` None ties the head to the embedding table."""
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight_name = weight_name
        self.weight = None

    def tensor_specs(self):
        if self.weight_name is None:
            return []
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, setup, tied_table=None):
        self.weight = tied_table if self.weight_name is None else setup.place(tensors[self.weight_name])

    def forward(self, rows, ctx):
        logits = ctx.buffer("logits", rows.shape[0], self.vocab_size, dtype="float32")
        ctx.ops.linear(rows, self.weight, None, logits)
        return logits
