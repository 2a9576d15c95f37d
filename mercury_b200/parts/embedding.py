"""Token embedding and the output head.

Embedding: a row lookup without scaling (mercury/model/qwen2.py:100, :109), written into
the float32 residual stream. Head: hidden times a [vocab, hidden] matrix, no bias
(mercury/model/qwen2.py:128-130, :145-150); logits are float32. A head is tied to the
embedding by naming the embedding's checkpoint tensor as its own weight: both parts then
get the same buffer from `PartSetup.place_named`.

Both are registered kinds ("lookup", "linear"), so a model description chooses them like
any other part; an embedding that scales its rows or a head with a bias or a soft cap is
another registered kind, not a change to the generic model.
"""

from __future__ import annotations

from .base import Embedding, Head, TensorSpec, register_embedding, register_head


class TokenEmbedding(Embedding):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight_name = weight_name
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, setup):
        self.table = setup.place_named(tensors, self.weight_name)

    def forward(self, token_ids, ctx):
        h = ctx.buffer("residual", token_ids.shape[0], self.hidden_size, dtype="float32")
        ctx.ops.embed(token_ids, self.table, h)
        return h


class LinearHead(Head):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight_name = weight_name
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, setup):
        self.weight = setup.place_named(tensors, self.weight_name)

    def forward(self, rows, ctx):
        logits = ctx.buffer("logits", rows.shape[0], self.vocab_size, dtype="float32")
        ctx.ops.linear(rows, self.weight, None, logits)
        return logits


register_embedding("lookup", TokenEmbedding)
register_head("linear", LinearHead)
