"""Python entry to eb_greedy_step: the tail of a greedy generation step in one launch."""
import torch

from ._lib import lib, check, dtype_code, ptr, stream_ptr, require_cuda


def greedy_step(logits, out_ids, tok, kv_state, counter, word_emb=None, pos_emb=None, hidden_out=None, vocab_start=0,
                add_pos=True):
    """logits [B, V] (last dim contiguous); out_ids [B, cols] int64; tok [B] int64 or None;
    kv_state int32[2] = (position just processed, column of the new token); counter int32[1],
    zero between calls.  With word_emb [rows, h] / pos_emb [P, h] given, hidden_out [B, h] (rows may
    be strided) receives the embedding of the new tokens at the next position; vocab_start is
    the first token id of word_emb (a slice of a vocabulary split over ranks), add_pos whether
    this rank adds the position embedding.  Advances kv_state by one."""
    require_cuda(logits, out_ids, tok, kv_state, counter, word_emb, pos_emb, hidden_out)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise RuntimeError("greedy_step: logits must be [batch, vocab] with a contiguous last dim")
    if out_ids.dtype != torch.int64 or out_ids.dim() != 2 or out_ids.stride(1) != 1 or (tok is not None and tok.dtype != torch.int64):
        raise RuntimeError("greedy_step: ids must be int64, out_ids [batch, columns]")
    if kv_state.dtype != torch.int32 or counter.dtype != torch.int32:
        raise RuntimeError("greedy_step: kv_state and counter must be int32")
    B, V = logits.shape
    hidden = 0
    if word_emb is not None:
        if not (word_emb.dtype == pos_emb.dtype == hidden_out.dtype):
            raise RuntimeError("greedy_step: embedding tables and output must share a dtype")
        if not (word_emb.is_contiguous() and pos_emb.is_contiguous() and hidden_out.stride(-1) == 1):
            raise RuntimeError("greedy_step: embedding tables must be contiguous")
        hidden = word_emb.shape[1]
        hidden_out = hidden_out.view(B, hidden) if hidden_out.dim() != 2 else hidden_out
    check(lib().eb_greedy_step(ptr(logits), logits.stride(0), B, V, dtype_code(logits.dtype), ptr(out_ids), out_ids.stride(0),
                               out_ids.shape[1], ptr(tok), ptr(kv_state), ptr(word_emb), int(vocab_start),
                               word_emb.shape[0] if word_emb is not None else 0, ptr(pos_emb),
                               pos_emb.shape[0] if pos_emb is not None else 0, 1 if add_pos else 0, hidden,
                               dtype_code(word_emb.dtype) if word_emb is not None else 0, ptr(hidden_out),
                               hidden_out.stride(0) if hidden_out is not None else 0, ptr(counter), stream_ptr()), "greedy_step")
