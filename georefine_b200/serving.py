"""nn.Module adapters over a compressed weight.

Mirrors ``BctxLinear`` / ``BctxEmbedding`` of
``context-runtime/georefine_context_runtime/bitexact_context_serving.py:346-400``: same constructor, counters
and attributes, not part of ``state_dict``.  ``forward`` calls the fused kernel instead of decoding the whole
weight and running a dense matmul; ``.weight`` still decodes transiently for helpers that want a dense tensor.
"""
from __future__ import annotations

import torch
from torch import nn


class ContextServingError(RuntimeError):
    pass


class BctxLinear(nn.Module):
    """Linear whose weight stays compressed; the product never materialises a dense copy."""

    def __init__(self, tensor, bias=None):
        super().__init__()
        if len(tensor.shape) != 2:
            raise ContextServingError("linear BCTX weight must be rank two")
        self.context_weight = tensor
        self.out_features, self.in_features = map(int, tensor.shape)
        self.forward_calls = 0
        self.weight_materializations = 0
        self.register_parameter("bias", bias)

    @property
    def weight(self):
        self.weight_materializations += 1
        return self.context_weight.decode()

    def forward(self, x):
        self.forward_calls += 1
        bias = None if self.bias is None else self.bias.to(torch.bfloat16)
        return self.context_weight.linear(x, bias=bias)


class BctxEmbedding(nn.Module):
    """Embedding table that stays compressed; rows are decoded by indexed gather."""

    def __init__(self, tensor, *, padding_idx=None):
        super().__init__()
        if len(tensor.shape) != 2:
            raise ContextServingError("embedding BCTX weight must be rank two")
        self.context_weight = tensor
        self.num_embeddings, self.embedding_dim = map(int, tensor.shape)
        self.padding_idx = padding_idx
        self.forward_calls = 0
        self.weight_materializations = 0

    @property
    def weight(self):
        self.weight_materializations += 1
        return self.context_weight.decode()

    def forward(self, input):
        self.forward_calls += 1
        return self.context_weight.gather_rows(input)
