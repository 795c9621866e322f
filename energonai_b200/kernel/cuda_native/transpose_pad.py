"""Padding remove/rebuild and head transposes with the reference's Python signatures
(energonai/kernel/cuda_native/transpose_pad.py:12-87).  Outputs are allocated with
torch.empty; the kernels write the zero rows themselves."""
import torch

from ..._lib import lib, check, dtype_code, ptr, stream_ptr, require_cuda


def _int32(t, name):
    # The reference reads these with data_ptr<int>() (transpose_pad_fusion_wrapper.cpp:48);
    # int64 tensors, which its own stale test passes, are converted instead of misread.
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t.contiguous()


def _float_dtype(t, what):
    if t.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"{what}: Datatype not implemented ({t.dtype})")


def transpose_pad(src, batch_size, max_seq_len, seq_len_list, head_num, size_per_head):
    """[1, sum_len, head_num, size_per_head] -> [batch, head_num, max_seq_len, size_per_head]."""
    require_cuda(src, seq_len_list)
    _float_dtype(src, "transpose_pad")
    src = src.contiguous()
    lens = _int32(seq_len_list, "seq_len_list")
    dst = torch.empty((batch_size, head_num, max_seq_len, size_per_head), dtype=src.dtype, device=src.device)
    check(lib().eb_transpose_pad(ptr(src), ptr(dst), batch_size, max_seq_len, ptr(lens), head_num, size_per_head,
                                 dtype_code(src.dtype), stream_ptr()), "transpose_pad")
    return dst


def transpose_depad(src, batch_size, sum_seq, max_seq_len, seq_len_list, head_num, size_per_head):
    """[batch, head_num, max_seq_len, size_per_head] -> [1, sum_seq, head_num, size_per_head]."""
    require_cuda(src, seq_len_list)
    _float_dtype(src, "transpose_depad")
    src = src.contiguous()
    lens = _int32(seq_len_list, "seq_len_list")
    sum_seq = int(sum_seq)
    dst = torch.empty((1, sum_seq, head_num, size_per_head), dtype=src.dtype, device=src.device)
    check(lib().eb_transpose_depad(ptr(src), ptr(dst), batch_size, sum_seq, max_seq_len, ptr(lens), head_num,
                                   size_per_head, dtype_code(src.dtype), stream_ptr()), "transpose_depad")
    return dst


def depad(src, batch_size, seq_lens):
    """Concatenate the valid prefix of every sequence along dim 1
    (energonai/kernel/cuda_native/transpose_pad.py:30-37).  Pure tensor indexing in the
    reference as well; kept for API completeness."""
    return torch.cat([src[i:i + 1, 0:int(seq_lens[i]), :] for i in range(batch_size)], dim=1)


def ft_build_padding_offsets(seq_lens, batch_size, max_seq_len, valid_word_num, tmp_mask_offset):
    require_cuda(seq_lens, valid_word_num, tmp_mask_offset)
    if valid_word_num.dtype != torch.int32 or tmp_mask_offset.dtype != torch.int32:
        raise RuntimeError("ft_build_padding_offsets: outputs must be int32 tensors")
    if not (valid_word_num.is_contiguous() and tmp_mask_offset.is_contiguous()):
        raise RuntimeError("ft_build_padding_offsets: outputs must be contiguous")
    if tmp_mask_offset.numel() < batch_size * max_seq_len:
        raise RuntimeError("ft_build_padding_offsets: tmp_mask_offset needs batch_size*max_seq_len entries")
    lens = _int32(seq_lens, "seq_lens")
    check(lib().eb_build_padding_offsets(ptr(lens), batch_size, max_seq_len, ptr(valid_word_num), ptr(tmp_mask_offset),
                                         stream_ptr()), "ft_build_padding_offsets")


def ft_remove_padding(src, tmp_mask_offset, mask_offset, valid_word_num, hidden_dim):
    require_cuda(src, tmp_mask_offset, mask_offset)
    _float_dtype(src, "ft_remove_padding")
    src = src.contiguous()
    valid_word_num = int(valid_word_num)
    if mask_offset.dtype != torch.int32 or tmp_mask_offset.dtype != torch.int32:
        raise RuntimeError("ft_remove_padding: offsets must be int32 tensors")
    if valid_word_num > min(tmp_mask_offset.numel(), mask_offset.numel()) or valid_word_num * hidden_dim > src.numel():
        raise RuntimeError("ft_remove_padding: valid_word_num exceeds the given tensors")
    dst = torch.empty((1, valid_word_num, hidden_dim), dtype=src.dtype, device=src.device)
    check(lib().eb_remove_padding(ptr(src), ptr(dst), ptr(tmp_mask_offset), ptr(mask_offset), valid_word_num, hidden_dim,
                                  dtype_code(src.dtype), stream_ptr()), "ft_remove_padding")
    return dst


def ft_rebuild_padding(src, mask_offset, valid_word_num, hidden_dim, batch_size, max_seq_len):
    require_cuda(src, mask_offset)
    _float_dtype(src, "ft_rebuild_padding")
    src = src.contiguous()
    valid_word_num = int(valid_word_num)
    if mask_offset.dtype != torch.int32:
        raise RuntimeError("ft_rebuild_padding: mask_offset must be an int32 tensor")
    if valid_word_num > mask_offset.numel() or valid_word_num * hidden_dim > src.numel():
        raise RuntimeError("ft_rebuild_padding: valid_word_num exceeds the given tensors")
    dst = torch.empty((batch_size, max_seq_len, hidden_dim), dtype=src.dtype, device=src.device)
    check(lib().eb_rebuild_padding(ptr(src), ptr(dst), ptr(mask_offset), valid_word_num, hidden_dim, batch_size,
                                   max_seq_len, dtype_code(src.dtype), 1, stream_ptr()), "ft_rebuild_padding")
    return dst


def ft_transpose_rebuild_padding(Q, K, V, q_buf, k_buf, v_buf, batch_size, seq_len, head_num, size_per_head,
                                 valid_word_num, mask_offset):
    """Scatters into the caller's buffers and returns None, like the reference: rows of
    padding tokens keep whatever the caller put there (its callers pre-zero them)."""
    require_cuda(Q, K, V, q_buf, k_buf, v_buf, mask_offset)
    _float_dtype(Q, "ft_transpose_rebuild_padding")
    for t in (q_buf, k_buf, v_buf):
        if not t.is_contiguous() or t.dtype != Q.dtype:
            raise RuntimeError("ft_transpose_rebuild_padding: output buffers must be contiguous and of the input dtype")
        if t.numel() < batch_size * seq_len * head_num * size_per_head:
            raise RuntimeError("ft_transpose_rebuild_padding: output buffer too small")
    Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
    valid_word_num = int(valid_word_num)
    if mask_offset.dtype != torch.int32 or valid_word_num > mask_offset.numel():
        raise RuntimeError("ft_transpose_rebuild_padding: mask_offset must be int32 with valid_word_num entries")
    check(lib().eb_transpose_rebuild_padding(ptr(Q), ptr(K), ptr(V), ptr(q_buf), ptr(k_buf), ptr(v_buf), batch_size,
                                             seq_len, head_num, size_per_head, valid_word_num, ptr(mask_offset),
                                             dtype_code(Q.dtype), 0, stream_ptr()), "ft_transpose_rebuild_padding")


def ft_transpose_remove_padding(src, valid_word_num, batch_size, seq_len, head_num, size_per_head, mask_offset):
    require_cuda(src, mask_offset)
    _float_dtype(src, "ft_transpose_remove_padding")
    src = src.contiguous()
    valid_word_num = int(valid_word_num)
    if mask_offset.dtype != torch.int32 or valid_word_num > mask_offset.numel():
        raise RuntimeError("ft_transpose_remove_padding: mask_offset must be int32 with valid_word_num entries")
    dst = torch.empty((1, valid_word_num, head_num * size_per_head), dtype=src.dtype, device=src.device)
    check(lib().eb_transpose_remove_padding(ptr(src), ptr(dst), valid_word_num, batch_size, seq_len, head_num,
                                            size_per_head, ptr(mask_offset), dtype_code(src.dtype), stream_ptr()),
          "ft_transpose_remove_padding")
    return dst
