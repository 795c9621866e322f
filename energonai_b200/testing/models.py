"""Engine fixture in the spirit of the reference's BoringModel (energonai/testing/models.py:8-38):
an all-ones 4x4 linear layer with an all-ones bias, split row-parallel over the tensor-parallel
group, so every stage maps x to 4x + 1 whatever the number of ranks.  It is plain torch (the
engine under test is transport and batching, not kernels) and runs on CPU or GPU."""
import torch
import torch.nn as nn

from ..tp import get_tp


class BoringModel(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        tp = get_tp()
        self.weight = nn.Parameter(torch.ones(4, 4 // tp.world_size))     # this rank's input columns
        self.bias = nn.Parameter(torch.ones(4))

    def forward(self, x):
        tp = get_tp()
        n = 4 // tp.world_size
        part = x[..., tp.rank * n:(tp.rank + 1) * n] @ self.weight.t()
        return tp.all_reduce(part) + self.bias


def get_correct_output(x: torch.Tensor, pp_world_size: int = 1) -> torch.Tensor:
    for _ in range(pp_world_size):
        x = x * 4 + 1
    return x
