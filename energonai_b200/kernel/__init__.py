"""Kernel API with the call signatures of the reference's `energonai.kernel`
(energonai/kernel/__init__.py:1-10), backed by the sm_100a C-ABI library."""
from .cuda_native import transpose_pad, transpose_depad, depad, scale_mask_softmax
from .cuda_native import (ft_build_padding_offsets, ft_remove_padding, ft_rebuild_padding,
                          ft_transpose_remove_padding, ft_transpose_rebuild_padding)
from .cuda_native import linear, find_algo
from .cuda_native import LayerNorm

__all__ = [
    "transpose_pad", "transpose_depad", "depad", "scale_mask_softmax", "ft_build_padding_offsets", "ft_remove_padding",
    "ft_rebuild_padding", "ft_transpose_remove_padding", "ft_transpose_rebuild_padding", "linear", "find_algo",
    "LayerNorm",
]
