"""Tensor-parallel-size-1 restatement of the Megatron 1-D layers the reference uses.

Column-parallel: y = x W^T + b with W split on dim 0 (no communication).
Row-parallel:    y = allreduce(x_r W_r^T) + b with W split on dim 1, bias added once.
With one rank both are a plain linear layer.
"""
import torch
from torch import nn
import torch.nn.functional as F


class Linear1D_Col(nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=None, gather_output=False, **kw):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


class Linear1D_Row(nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=None, parallel_input=True, **kw):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        y = F.linear(x, self.weight)
        return y if self.bias is None else y + self.bias


class LayerNorm1D(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, dtype=None):
        super().__init__()
        self.module = nn.LayerNorm(normalized_shape, eps=eps, dtype=dtype)

    def forward(self, x):
        return self.module(x)


class VocabParallelEmbedding1D(nn.Embedding):
    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, dtype=None, **kw):
        super().__init__(num_embeddings, embedding_dim, padding_idx=padding_idx, dtype=dtype)


class Classifier1D(nn.Module):
    def __init__(self, in_features, num_classes, weight=None, bias=True, dtype=None, **kw):
        super().__init__()
        if weight is not None:
            self.weight = weight
        else:
            self.weight = nn.Parameter(torch.empty(num_classes, in_features, dtype=dtype))
            nn.init.normal_(self.weight, std=0.02)
        self.bias = nn.Parameter(torch.zeros(num_classes, dtype=dtype)) if bias else None

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


class VocabParallelClassifier1D(Classifier1D):
    def __init__(self, in_features, num_classes, weight=None, bias=True, dtype=None, gather_output=False, **kw):
        super().__init__(in_features, num_classes, weight=weight, bias=bias, dtype=dtype)
