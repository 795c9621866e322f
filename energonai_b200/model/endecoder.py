"""Block1D with the reference's constructor and forward signature
(energonai/model/endecoder.py:11-70): norm1 -> attention -> +residual -> norm2 -> MLP ->
+residual, pre-LN or the reference's post-LN variant (residual taken after the norm).
The residual additions run inside the epilogues of the two row-parallel GEMMs."""
import os
from typing import Callable

import torch
from torch import dtype, nn

from ..nn import LayerNorm1D, can_fold
from .attention import MultiHeadAttention1D
from .mlp import MLP1D


class Block1D(nn.Module):
    def __init__(self,
                 hidden_size: int,
                 num_heads: int,
                 mlp_ratio: float,
                 activation: Callable = nn.functional.gelu,
                 layernorm_epsilon: float = 1e-5,
                 dtype: dtype = torch.float16,
                 bias: bool = True,
                 apply_post_layernorm: bool = False,
                 max_seq_len: int = 512,
                 fused_qkv: bool = True,
                 is_decoder: bool = True,
                 disable_past_cache=False) -> None:
        super().__init__()
        self.apply_post_layernorm = apply_post_layernorm
        self.disable_past_cache = disable_past_cache
        # generation steps: norm1 / norm2 are evaluated inside the QKV / FC1 GEMMs (pre-LN only)
        self.fold_layernorm = os.environ.get("EB_LN_FOLD", "1") != "0"
        self.norm1 = LayerNorm1D(hidden_size, eps=layernorm_epsilon, dtype=dtype)
        self.attn = MultiHeadAttention1D(hidden_size=hidden_size, num_heads=num_heads, bias=bias, dtype=dtype,
                                         max_seq_len=max_seq_len, fused_qkv=fused_qkv, is_decoder=is_decoder,
                                         disable_past_cache=disable_past_cache)
        self.norm2 = LayerNorm1D(hidden_size, eps=layernorm_epsilon, dtype=dtype)
        self.mlp = MLP1D(hidden_size=hidden_size, mlp_ratio=mlp_ratio, activation=activation, dtype=dtype, bias=bias,
                         disable_past_cache=disable_past_cache)

    def forward(self, hidden_states, attention_mask=None, first_cache=False, seq_lens=None, kv_state=None):
        """Prompt pass (first_cache=True, or no cache): [batch, seq, hidden] -> same shape.
        Generation step: only the last position of the input is used and [batch, 1, hidden] is
        returned (a caller may pass either the whole sequence, as the reference's generation
        loop does, or just the new position)."""
        if not (self.disable_past_cache or first_cache):
            hidden_states = hidden_states[:, -1:, :]
            if not self.apply_post_layernorm and can_fold(hidden_states.shape[0], hidden_states.dtype, self.fold_layernorm):
                hidden_states = self.attn(hidden_states, attention_mask=attention_mask, first_cache=False,
                                          residual=hidden_states, kv_state=kv_state, fold_norm=self.norm1)
                return self.mlp(hidden_states, first_cache=True, residual=hidden_states, fold_norm=self.norm2)
        # Prompt-sized sums of a tensor-parallel group may stay in the exchange's own buffers (two
        # alternate): the attention output is consumed by norm2 and as the MLP's residual, the
        # MLP output by the next block's norm1 and residual, both before the buffer comes round.
        normed = self.norm1(hidden_states)
        residual = normed if self.apply_post_layernorm else hidden_states
        hidden_states = self.attn(normed, attention_mask=attention_mask, first_cache=first_cache, residual=residual,
                                  kv_state=kv_state, transient_ok=True)
        normed = self.norm2(hidden_states)
        residual = normed if self.apply_post_layernorm else hidden_states
        return self.mlp(normed, first_cache=True, residual=residual, transient_ok=True)
