"""Embedding1D with the reference's interface (energonai/model/embedding.py:9-57): word plus
learned position embeddings, positions = arange over the padded sequence (no offset), optional
token-type embeddings.  `past_key_values_length` shifts the positions, which is what a
generation step that embeds only the new token needs."""
import torch
from torch import nn, dtype
from torch.nn import Embedding


class Embedding1D(nn.Module):
    def __init__(self, hidden_size: int, vocab_size: int, max_seq_len: int, num_tokentypes: int = 0,
                 padding_idx: int = 0, dtype: dtype = None, vocab_parallel: bool = False) -> None:
        super().__init__()
        if vocab_parallel:
            from ..nn import VocabParallelEmbedding1D
            self.word_embeddings = VocabParallelEmbedding1D(vocab_size, hidden_size, padding_idx=padding_idx, dtype=dtype)
        else:
            self.word_embeddings = Embedding(vocab_size, hidden_size, padding_idx=padding_idx).to(dtype=dtype)
        self.position_embeddings = Embedding(max_seq_len, hidden_size).to(dtype=dtype)
        self.tokentype_embeddings = Embedding(num_tokentypes, hidden_size).to(dtype=dtype) if num_tokentypes > 0 else None

    @property
    def word_embedding_weight(self):
        return self.word_embeddings.weight

    def forward(self, input_ids, position_ids=None, tokentype_ids=None, past_key_values_length: int = 0):
        seq_length = input_ids.size(1)
        if position_ids is None:
            position_ids = torch.arange(past_key_values_length, past_key_values_length + seq_length, dtype=torch.long,
                                        device=input_ids.device).unsqueeze(0)
        x = self.word_embeddings(input_ids) + self.position_embeddings(position_ids)
        if self.tokentype_embeddings is not None and tokentype_ids is not None:
            x = x + self.tokentype_embeddings(tokentype_ids)
        return x
