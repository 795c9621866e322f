from .transpose_pad import transpose_pad, transpose_depad, depad
from .transpose_pad import (ft_build_padding_offsets, ft_remove_padding, ft_rebuild_padding,
                            ft_transpose_remove_padding, ft_transpose_rebuild_padding)
from .scale_mask_softmax import scale_mask_softmax
from .layer_norm import MixedFusedLayerNorm as LayerNorm
from .linear_func import linear, find_algo
