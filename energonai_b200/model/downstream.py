"""LMHead1D with the reference's interface (energonai/model/downstream.py:5-26): a bias-free
(by default) projection to the vocabulary on the tcgen05 GEMM, logits in fp32; with
vocab_parallel every rank computes its slice of the vocabulary and the slices are gathered."""
import torch
from torch import dtype, nn

from ..gemm import gemm
from ..nn import FoldCache


class _Classifier(nn.Module):
    def __init__(self, in_features, num_classes, weight=None, bias=False, dtype=None):
        super().__init__()
        self.weight = weight if weight is not None else nn.Parameter(torch.empty(num_classes, in_features, dtype=dtype))
        if weight is None:
            nn.init.normal_(self.weight, std=0.02)
        self.bias = nn.Parameter(torch.zeros(num_classes, dtype=dtype)) if bias else None
        self._fold = FoldCache()

    def forward(self, x, fold_norm=None):
        """fold_norm: the final LayerNorm1D; x is then its un-normalised input (generation steps)."""
        x2 = x.reshape(-1, x.shape[-1])
        if fold_norm is not None:
            w_f, colsum, bias32, eps = self._fold.get(self.weight, self.bias, fold_norm)
            y = gemm(x2, w_f, out_dtype=torch.float32, static_weight=True, ln_fold=(colsum, bias32, eps))
        else:
            y = gemm(x2, self.weight, bias=self.bias, out_dtype=torch.float32, static_weight=True)
        return y.view(*x.shape[:-1], self.weight.shape[0])


class LMHead1D(nn.Module):
    def __init__(self, hidden_size: int, vocab_size: int, word_embedding_weight: nn.Parameter = None,
                 bias: bool = False, dtype: dtype = None, vocab_parallel: bool = False) -> None:
        super().__init__()
        self.vocab_parallel = vocab_parallel
        if vocab_parallel:
            from ..nn import VocabParallelClassifier1D
            self.dense = VocabParallelClassifier1D(hidden_size, vocab_size, bias=bias, dtype=dtype, gather_output=True)
        else:
            self.dense = _Classifier(hidden_size, vocab_size, word_embedding_weight, bias=bias, dtype=dtype)

    @property
    def weight(self):
        return self.dense.weight

    def forward(self, x, fold_norm=None):
        return self.dense(x, fold_norm=fold_norm)
