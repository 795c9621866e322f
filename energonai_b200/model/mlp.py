"""MLP1D with the reference's constructor and forward signature (energonai/model/mlp.py:8-51):
column-parallel FC1 with the activation fused into the GEMM epilogue, row-parallel FC2.
Generation steps process and return only the new position (see attention.py)."""
from typing import Callable, Optional

import torch
from torch import dtype, nn

from ..nn import Linear1D_Col, Linear1D_Row


def gelu_impl(x):
    """OpenAI's tanh GELU (energonai/model/model_factory.py:32-35), used as an activation tag."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)))


def activation_code(fn):
    """Maps the callables the reference passes as `activation` to an epilogue code."""
    name = getattr(fn, "__name__", str(fn))
    if fn is nn.functional.relu or name == "relu":
        return "relu"
    if name in ("gelu_impl", "gelu_tanh", "gelu_new"):
        return "gelu_tanh"
    if fn is nn.functional.gelu or name == "gelu":
        return "gelu"
    raise RuntimeError(f"MLP1D: activation {name!r} has no fused epilogue (relu, gelu, gelu_impl are supported)")


class MLP1D(nn.Module):

    def __init__(self,
                 hidden_size: int,
                 mlp_ratio: float,
                 activation: Callable,
                 dtype: dtype = torch.float16,
                 bias: bool = True,
                 disable_past_cache=False):
        super().__init__()
        self.disable_past_cache = disable_past_cache
        intermediate_dim = int(hidden_size * mlp_ratio)
        self.dense_1 = Linear1D_Col(hidden_size, intermediate_dim, bias=bias, dtype=dtype, gather_output=False)
        self.activation = activation
        self.act_code = activation_code(activation)
        self.dense_2 = Linear1D_Row(intermediate_dim, hidden_size, bias=bias, dtype=dtype, parallel_input=True)

    def forward(self, hidden_states, first_cache: Optional[bool] = True, residual=None, fold_norm=None, transient_ok=False):
        """fold_norm: see Linear1D_Col.forward (hidden_states is then the un-normalised input)."""
        if not (self.disable_past_cache or first_cache):
            hidden_states = hidden_states[:, -1:, :]
            residual = residual[:, -1:, :] if residual is not None else None
        inter = self.dense_1(hidden_states, act=self.act_code, fold_norm=fold_norm)
        return self.dense_2(inter, residual=residual, transient_ok=transient_ok)
