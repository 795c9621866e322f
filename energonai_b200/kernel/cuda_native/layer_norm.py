"""Fused LayerNorm module with the reference's interface
(energonai/kernel/cuda_native/layer_norm.py:48-78).  Forward only: this package is an
inference path, so the autograd backward of the reference (training) is not provided and
asking for it raises."""
import numbers

import torch
from torch.nn import init
from torch.nn.parameter import Parameter

from ..._lib import lib, check, dtype_code, ptr, stream_ptr, require_cuda


def layer_norm_forward(x, weight, bias, eps, residual=None, add_bias=None, return_sum=False, return_stats=False,
                       out_dtype=None):
    """y = LayerNorm(x (+ residual) (+ add_bias)) over the last dimension.

    Returns y, optionally followed by the pre-normalisation sum (in x's dtype) and
    (mean, invvar) fp32 per row, matching forward_affine's outputs
    (csrc/layer_norm_cuda.cpp:82-103)."""
    require_cuda(x, weight, bias, residual, add_bias)
    x = x.contiguous()
    n2 = x.shape[-1]
    n1 = x.numel() // n2 if n2 else 0
    out_dtype = out_dtype or (weight.dtype if weight is not None else x.dtype)
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    if residual is not None:
        residual = residual.contiguous()
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise RuntimeError("layer_norm: residual must match the input's shape and dtype")
    if add_bias is not None and (add_bias.numel() != n2 or add_bias.dtype != x.dtype):
        raise RuntimeError("layer_norm: add_bias must have n2 entries of the input dtype")
    if weight is not None and (weight.numel() != n2 or bias.numel() != n2 or weight.dtype != out_dtype or bias.dtype != out_dtype):
        raise RuntimeError("layer_norm: weight/bias must have n2 entries of the output dtype")
    total = torch.empty_like(x) if return_sum else None
    mean = torch.empty(n1, dtype=torch.float32, device=x.device) if return_stats else None
    invvar = torch.empty(n1, dtype=torch.float32, device=x.device) if return_stats else None
    check(lib().eb_layer_norm_fwd(ptr(y), ptr(mean), ptr(invvar), ptr(x), ptr(residual), ptr(add_bias), ptr(total),
                                  ptr(weight), ptr(bias), n1, n2, float(eps), dtype_code(x.dtype), dtype_code(out_dtype),
                                  stream_ptr()), "layer_norm_fwd")
    out = (y,)
    if return_sum:
        out += (total,)
    if return_stats:
        out += (mean, invvar)
    return out[0] if len(out) == 1 else out


class MixedFusedLayerNorm(torch.nn.Module):

    def __init__(self, normalized_shape, eps=1e-5, device=None, dtype=None):
        super().__init__()
        lib()   # fail at construction, like the reference, when the native library is absent
        if isinstance(normalized_shape, numbers.Integral):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = torch.Size(normalized_shape)
        self.eps = eps
        self.weight = Parameter(torch.empty(*normalized_shape, device=device, dtype=dtype))
        self.bias = Parameter(torch.empty(*normalized_shape, device=device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self):
        init.ones_(self.weight)
        init.zeros_(self.bias)

    def forward(self, input):
        if torch.is_grad_enabled() and (input.requires_grad or self.weight.requires_grad):
            raise RuntimeError("MixedFusedLayerNorm is forward-only here; call it under torch.inference_mode() "
                               "or torch.no_grad() (the reference's backward_affine is a training path)")
        if tuple(input.shape[-len(self.normalized_shape):]) != tuple(self.normalized_shape):
            raise RuntimeError(f"Given normalized_shape={list(self.normalized_shape)}, expected input with shape "
                               f"[*, {', '.join(map(str, self.normalized_shape))}], but got input of size{list(input.shape)}")
        n2 = self.weight.numel()
        return layer_norm_forward(input.reshape(-1, n2), self.weight.detach().reshape(-1), self.bias.detach().reshape(-1),
                                  self.eps).view(input.shape)

    def __repr__(self):
        return f'MixedFusedLayerNorm(normalized_shape={self.normalized_shape}, eps={self.eps})'
