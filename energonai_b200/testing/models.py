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


class EchoGenerator(nn.Module):
    """Stand-in for a generation model behind the engine: takes the keyword arguments a
    PipelineModel takes and returns [batch, max_tokens] token ids, each row its (padded) prompt
    followed by tokens that depend only on that row's own unpadded prompt, so the answer to a
    request does not depend on which other requests it was batched with."""

    def forward(self, input_ids=None, attention_mask=None, max_tokens=0, top_k=None, top_p=None, temperature=None):
        width = input_ids.shape[1]
        seed = (input_ids * attention_mask).sum(1, keepdim=True)
        steps = torch.arange(max_tokens - width, device=input_ids.device)[None, :]
        return torch.cat([input_ids, expected_new_tokens(seed, steps)], 1)


def expected_new_tokens(seed, steps):
    return 2 + (seed * 7 + steps * 13) % 997


class FlakyModel(nn.Module):
    """4x + 1 like BoringModel at tensor-parallel size 1, except for two marker inputs: a first
    element of -1 raises (a request the model rejects), a first element of -2 ends the worker
    process at once (a crashed worker).  A first element of -3 makes `health()` report a fault
    from then on, which is how a worker learns that a bounded device-side wait ran out (made on
    the host here; no GPU is involved).  Used to test what the engine tells its callers."""

    def __init__(self, fail_at_start: bool = False) -> None:
        super().__init__()
        if fail_at_start:
            raise RuntimeError("model_fn failed on purpose")
        self.fault = None

    def health(self):
        return self.fault

    def forward(self, x):
        marker = float(x.reshape(-1)[0])
        if marker == -3.0:
            self.fault = "a wait on a tensor-parallel peer ran out (made up by the test)"
        if marker == -1.0:
            raise ValueError("request rejected by the model")
        if marker == -2.0:
            import os
            os._exit(7)
        return x * 4 + 1
