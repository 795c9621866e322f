"""The 1-D tensor-parallel building blocks the reference imports from colossalai
(Linear1D_Col, Linear1D_Row, LayerNorm1D; used at energonai/model/attention.py:29-37,
mlp.py:20-22, endecoder.py:28,39), on the tcgen05 GEMM and the fused LayerNorm kernel.

Semantics (Megatron 1-D):
  Linear1D_Col  y_r = x W_r^T + b_r,  W split on dim 0 (each rank owns out/t rows), no
                communication unless gather_output.
  Linear1D_Row  y = allreduce_r(x_r W_r^T) + b,  W split on dim 1 (each rank owns in/t
                columns), bias added once after the reduction.
  LayerNorm1D   replicated affine LayerNorm; the parameters live on a child called `module`,
                which gives the reference's state_dict names (norm1.module.weight ...).
"""
import torch
from torch import nn

from .gemm import gemm, fold_layernorm, LN_FOLD_MAX_ROWS
from .kernel.cuda_native.layer_norm import layer_norm_forward
from .tp import get_tp, divide


def _flat(x):
    return x.reshape(-1, x.shape[-1])


def tensor_version(t):
    """In-place modification counter of a tensor; tensors created under inference_mode have none."""
    try:
        return t._version
    except RuntimeError:
        return -1


class FoldCache:
    """Keeps (w_folded, colsum, bias32) of fold_layernorm() for one (weight, LayerNorm) pair and
    rebuilds it when any of the tensors involved was reassigned or written in place."""

    def __init__(self):
        self.key, self.val = None, None

    def get(self, w, b, norm, versions=()):
        g, be = norm.module.weight, norm.module.bias
        key = (w.data_ptr(), tensor_version(w), None if b is None else (b.data_ptr(), tensor_version(b)), g.data_ptr(),
               tensor_version(g), be.data_ptr(), tensor_version(be), tuple(versions))
        if key != self.key:
            self.val = fold_layernorm(w, b, g, be) + (norm.eps,)
            self.key = key
        return self.val


def can_fold(rows, dtype, enabled=True):
    """A LayerNorm can be folded into the projection that follows it for generation-step shapes."""
    return enabled and rows <= LN_FOLD_MAX_ROWS and dtype in (torch.float16, torch.bfloat16)


class Linear1D_Col(nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=None, gather_output=False, device=None):
        super().__init__()
        tp = get_tp()
        self.in_features, self.out_features, self.gather_output = in_features, out_features, gather_output
        self.out_per_rank = divide(out_features, tp.world_size)
        self.weight = nn.Parameter(torch.empty(self.out_per_rank, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(self.out_per_rank, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)
        self._fold = FoldCache()

    def forward(self, x, act=None, fold_norm=None):
        """fold_norm: the LayerNorm1D whose output this projection would consume; x is then that
        LayerNorm's INPUT and the normalisation happens inside the GEMM (generation steps)."""
        if fold_norm is not None:
            w_f, colsum, bias32, eps = self._fold.get(self.weight, self.bias, fold_norm)
            y = gemm(_flat(x), w_f, act=act, static_weight=True, ln_fold=(colsum, bias32, eps))
        else:
            y = gemm(_flat(x), self.weight, bias=self.bias, act=act, static_weight=True)
        y = y.view(*x.shape[:-1], self.out_per_rank)
        return get_tp().all_gather_last_dim(y) if self.gather_output else y


class Linear1D_Row(nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=None, parallel_input=True, device=None):
        super().__init__()
        tp = get_tp()
        self.in_features, self.out_features = in_features, out_features
        self.in_per_rank = divide(in_features, tp.world_size)
        self.weight = nn.Parameter(torch.empty(out_features, self.in_per_rank, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x, residual=None, transient_ok=False):
        """x is this rank's slice of the input features.  Bias (and an optional residual) enter
        the sum exactly once: after the reduction (peer exchange), or in rank 0's GEMM epilogue
        before an NCCL all-reduce.  transient_ok: the caller consumes the result before the
        second-next row-parallel call, so a prompt-sized result may stay in the exchange's own
        buffer instead of being copied out."""
        tp = get_tp()
        x2 = _flat(x)
        if tp.peer is not None and tp.peer.fits(x2.shape[0], self.out_features):
            # generation steps: the all-reduce runs inside the GEMM epilogue over NVLink peer stores
            res = _flat(residual) if residual is not None else None
            y = gemm(x2, self.weight, bias=self.bias, residual=res, static_weight=True, peer=tp.peer)
            return y.view(*x.shape[:-1], self.out_features)
        if (tp.peer is not None and x2.dtype in (torch.float16, torch.bfloat16)
                and tp.peer.fits_bulk(x2.shape[0], self.out_features)):
            # prompt pass: reduce-scatter inside the GEMM epilogue, then one reduce + broadcast kernel
            res = _flat(residual) if residual is not None else None
            if res is not None and res.stride(-1) != 1:
                res = res.contiguous()
            y = tp.peer.row_parallel(x2, self.weight, bias=self.bias, residual=res)
            if not transient_ok:
                y = y.clone()
            return y.view(*x.shape[:-1], self.out_features)
        lead = tp.rank == 0
        res = _flat(residual) if (residual is not None and lead) else None
        y = gemm(_flat(x), self.weight, bias=self.bias if lead else None, residual=res, static_weight=True)
        tp.all_reduce(y)
        return y.view(*x.shape[:-1], self.out_features)


class VocabParallelEmbedding1D(nn.Module):
    """Word embedding with the vocabulary split over the tensor-parallel ranks (the colossalai
    layer the reference uses at energonai/model/embedding.py:21-23): rank r holds rows
    [r * V/t, (r+1) * V/t); ids owned by another rank contribute zero and the lookups are
    summed with one all-reduce."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, dtype=None, device=None):
        super().__init__()
        tp = get_tp()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.per_rank = divide(num_embeddings, tp.world_size)
        self.vocab_start = tp.rank * self.per_rank
        self.weight = nn.Parameter(torch.empty(self.per_rank, embedding_dim, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=0.02)
        if padding_idx is not None and self.vocab_start <= padding_idx < self.vocab_start + self.per_rank:
            with torch.no_grad():
                self.weight[padding_idx - self.vocab_start].zero_()

    def forward(self, ids):
        local = ids - self.vocab_start
        foreign = (local < 0) | (local >= self.per_rank)
        out = nn.functional.embedding(local.masked_fill(foreign, 0), self.weight)
        out = out.masked_fill(foreign.unsqueeze(-1), 0)
        return get_tp().all_reduce(out)


class VocabParallelClassifier1D(nn.Module):
    """Projection to a vocabulary split over the ranks (energonai/model/downstream.py:16): rank r
    computes the logits of its V/t classes; gather_output concatenates them on the last
    dimension in rank order."""

    def __init__(self, in_features, num_classes, bias=False, dtype=None, gather_output=True, device=None):
        super().__init__()
        tp = get_tp()
        self.in_features, self.num_classes, self.gather_output = in_features, num_classes, gather_output
        self.per_rank = divide(num_classes, tp.world_size)
        self.weight = nn.Parameter(torch.empty(self.per_rank, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(self.per_rank, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)
        self._fold = FoldCache()

    def forward(self, x, fold_norm=None):
        x2 = _flat(x)
        if fold_norm is not None:
            w_f, colsum, bias32, eps = self._fold.get(self.weight, self.bias, fold_norm)
            y = gemm(x2, w_f, out_dtype=torch.float32, static_weight=True, ln_fold=(colsum, bias32, eps))
        else:
            y = gemm(x2, self.weight, bias=self.bias, out_dtype=torch.float32, static_weight=True)
        y = y.view(*x.shape[:-1], self.per_rank)
        return get_tp().all_gather_last_dim(y) if self.gather_output else y


class _LayerNormParams(nn.Module):
    def __init__(self, n, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(n, dtype=dtype, device=device))


class LayerNorm1D(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, dtype=None, device=None):
        super().__init__()
        self.normalized_shape, self.eps = int(normalized_shape), eps
        self.module = _LayerNormParams(self.normalized_shape, dtype, device)

    def forward(self, x):
        return layer_norm_forward(_flat(x), self.module.weight, self.module.bias, self.eps).view(x.shape)
