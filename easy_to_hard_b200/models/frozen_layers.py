"""Embedding / RMSNorm / Linear whose weight is a *buffer*, not a Parameter.

The reference never trains embeddings, norms or (for policies) the LM head
(models/frozen_layers.py:35-187): only the block linears and the reward head are Parameters, so
the tensors that are replicated across tensor-parallel ranks need no gradient synchronisation
and take no optimizer state. The same split is kept here; the state-dict keys are unchanged
(``*.weight``), so checkpoints load into either flavour.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ..ops import reference as ref_ops


class FrozenEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, device=None, dtype=None):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        # set by models.tp.apply_tp when the table is sharded over the vocabulary
        self.vocab_start_index = None
        self.vocab_end_index = None
        self.register_buffer("weight", torch.empty(num_embeddings, embedding_dim, device=device,
                                                   dtype=dtype))

    def forward(self, idx: Tensor) -> Tensor:
        if self.vocab_start_index is None:
            return F.embedding(idx, self.weight)
        # vocab-parallel shard: rows outside [start, end) contribute zeros; the caller sums
        # the shards over the tensor-parallel group.
        outside = (idx < self.vocab_start_index) | (idx >= self.vocab_end_index)
        local = (idx - self.vocab_start_index).masked_fill(outside, 0)
        out = F.embedding(local, self.weight)
        return out.masked_fill(outside.unsqueeze(-1), 0.0)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}, frozen"


class FrozenRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.register_buffer("weight", torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        return ref_ops.rmsnorm(x, self.weight, self.eps)


class FrozenLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("weight", torch.empty(out_features, in_features, device=device,
                                                   dtype=dtype))

    def forward(self, x: Tensor) -> Tensor:
        return F.linear(x, self.weight)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, frozen"
