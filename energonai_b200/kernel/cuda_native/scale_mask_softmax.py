"""scale_mask_softmax with the reference's signature
(energonai/kernel/cuda_native/scale_mask_softmax.py:10-13)."""
import torch

from ..._lib import lib, check, dtype_code, ptr, stream_ptr, require_cuda, SM_CAUSAL


def scale_mask_softmax(batch_size, batch_seq_len, head_num, src, seq_len_list, *, flags=SM_CAUSAL, scale=1.0):
    """In-place causal, length-masked softmax over src [batch, head_num, seq, seq]; returns
    the (contiguous) tensor it wrote, like the reference.  The keyword arguments are
    extensions: the reference behaviour is flags=SM_CAUSAL, scale=1.0 (it applies no scale)."""
    require_cuda(src, seq_len_list)
    if src.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError("scale_mask_softmax: Datatype not implemented")
    src = src.contiguous()
    if src.numel() < batch_size * head_num * batch_seq_len * batch_seq_len:
        raise RuntimeError("scale_mask_softmax: src is smaller than batch*head*seq*seq")
    lens = seq_len_list if seq_len_list.dtype == torch.int32 else seq_len_list.to(torch.int32)
    lens = lens.contiguous()
    if lens.numel() < batch_size:
        raise RuntimeError("scale_mask_softmax: seq_len_list has fewer than batch_size entries")
    check(lib().eb_scale_mask_softmax(ptr(src), ptr(lens), batch_size, batch_seq_len, head_num, dtype_code(src.dtype),
                                      flags, float(scale), stream_ptr()), "scale_mask_softmax")
    return src
