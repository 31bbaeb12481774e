"""Token embedding and output head.

Embedding: h0[t] = E[id_t] (python/lyapunov_engine/models/llama.py:172,205),
written straight into the 32-bit residual stream.  Head: logits = n W^T in
float32, for the wanted rows only (the reference computes every position and
keeps the last, python/lyapunov_engine/engine/llm_engine.py:272,289).  A tied
head is the embedding matrix itself, not a copy of it (the reference copies,
python/lyapunov_engine/models/weight_loader.py:102-109).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorDecl, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str):
        self.vocab_size, self.hidden_size, self.weight_name = int(vocab_size), int(hidden_size), weight_name
        self.weight = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.vocab_size, self.hidden_size))]

    def bind(self, get, runtime):
        self.weight = get(self.weight_name)
        self.runtime = runtime

    def forward(self, ctx):
        resid = ctx.workspace.get("resid", (ctx.num_tokens, self.hidden_size), torch.float32)
        ops.embed(resid, self.weight, ctx.token_ids, ctx.status)
        return resid


@register_head("linear_head")
class LinearHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, tied_to: str | None = None):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight_name, self.tied_to = weight_name, tied_to
        self.weight = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.vocab_size, self.hidden_size), alias_of=self.tied_to)]

    def bind(self, get, runtime):
        self.weight = get(self.weight_name)
        self.runtime = runtime

    def forward(self, normed, ctx):
        logits = ctx.workspace.get("logits", (normed.shape[0], self.vocab_size), torch.float32)
        ops.linear(logits, normed, self.weight, ctx.status)
        return logits
