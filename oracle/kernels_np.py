"""NumPy restatements of the reference CUDA kernels (test infrastructure; see oracle/__init__.py).

Every function follows the indexing of one `__global__` function of
energonai/kernel/cuda_native/csrc/ and cites it.  Integer results are exact; float results
are computed in float64/float32 and cast to the array dtype the way the kernel does.
"""
import numpy as np


# ---------------------------------------------------------------------------------------
# FasterTransformer-style padding kernels  (transpose_pad_fusion_kernel.cu)
# ---------------------------------------------------------------------------------------
def build_padding_offsets(seq_lens, batch_size, max_seq_len):
    """transpose_pad_fusion_kernel.cu:112-131 (build_sequence_length_padding_offset).

    For every valid token, in packed order, the number of padding slots that precede it
    in the padded [batch, max_seq_len] layout.  Returns (valid_word_num, tmp_mask_offset)
    where tmp_mask_offset has exactly valid_word_num entries (int32).
    """
    lens = np.asarray(seq_lens, dtype=np.int64)[:batch_size]
    pads_before = np.concatenate([[0], np.cumsum(max_seq_len - lens)[:-1]]) if batch_size else np.zeros(0)
    offsets = np.repeat(pads_before, lens).astype(np.int32)
    return int(lens.sum()), offsets


def remove_padding(src, tmp_mask_offset, valid_word_num):
    """transpose_pad_fusion_kernel.cu:142-155: tgt[k] = src[k + off[k]]; also copies
    tmp_mask_offset into mask_offset.  src is [batch*max_seq_len, n]."""
    off = np.asarray(tmp_mask_offset[:valid_word_num], dtype=np.int32)
    k = np.arange(valid_word_num)
    src2 = src.reshape(-1, src.shape[-1])
    return src2[k + off].copy(), off.copy()


def rebuild_padding(src, mask_offset, valid_word_num, batch_size, max_seq_len):
    """transpose_pad_fusion_kernel.cu:178-190 into a zero tensor
    (transpose_pad_fusion_wrapper.cpp:158): tgt[k + off[k]] = src[k]."""
    n = src.shape[-1]
    src2 = src.reshape(-1, n)
    tgt = np.zeros((batch_size * max_seq_len, n), dtype=src.dtype)
    k = np.arange(valid_word_num)
    tgt[k + np.asarray(mask_offset[:valid_word_num])] = src2[:valid_word_num]
    return tgt.reshape(batch_size, max_seq_len, n)


def transpose_rebuild_padding(Q, q_buf, batch_size, seq_len, head_num, size_per_head, valid_word_num, mask_offset):
    """transpose_pad_fusion_kernel.cu:213-236 for one of the three tensors: packed
    [valid, head, dim] -> q_buf[batch, head, seq, dim] at the padded position of each token.
    Rows of padding tokens in q_buf are not written (the caller pre-zeroes them)."""
    Qv = Q.reshape(-1, head_num, size_per_head)
    pos = np.arange(valid_word_num) + np.asarray(mask_offset[:valid_word_num])
    b, s = pos // seq_len, pos % seq_len
    q_buf[b, :, s, :] = Qv[:valid_word_num]
    return q_buf


def transpose_remove_padding(src, valid_word_num, batch_size, seq_len, head_num, size_per_head, mask_offset):
    """transpose_pad_fusion_kernel.cu:268-289: [batch, head, seq, dim] -> packed
    [1, valid, head*dim]."""
    pos = np.arange(valid_word_num) + np.asarray(mask_offset[:valid_word_num])
    b, s = pos // seq_len, pos % seq_len
    out = src.reshape(batch_size, head_num, seq_len, size_per_head)[b, :, s, :]
    return out.reshape(1, valid_word_num, head_num * size_per_head).copy()


# ---------------------------------------------------------------------------------------
# TurboTransformers-style transposes  (transpose_pad_fusion_kernel.cu:8-96)
# ---------------------------------------------------------------------------------------
def transpose_pad(src, batch_size, max_seq_len, seq_lens, head_num, size_per_head):
    """transpose_pad_fusion_kernel.cu:58-84: packed [1, sum_len, head, dim] ->
    [batch, head, max_seq_len, dim], zero where seq position >= seq_lens[b]."""
    lens = np.asarray(seq_lens, dtype=np.int64)[:batch_size]
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    src3 = src.reshape(-1, head_num, size_per_head)
    dst = np.zeros((batch_size, head_num, max_seq_len, size_per_head), dtype=src.dtype)
    for b in range(batch_size):
        L = int(lens[b])
        dst[b, :, :L, :] = src3[starts[b]:starts[b] + L].transpose(1, 0, 2)
    return dst


def transpose_depad(src, batch_size, sum_seq, max_seq_len, seq_lens, head_num, size_per_head):
    """transpose_pad_fusion_kernel.cu:8-35 into zeros({1,sum_seq,head,dim})
    (transpose_pad_fusion_wrapper.cpp:70): [batch, head, seq, dim] -> packed."""
    lens = np.asarray(seq_lens, dtype=np.int64)[:batch_size]
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    src4 = src.reshape(batch_size, head_num, max_seq_len, size_per_head)
    dst = np.zeros((1, int(sum_seq), head_num, size_per_head), dtype=src.dtype)
    for b in range(batch_size):
        L = int(lens[b])
        dst[0, starts[b]:starts[b] + L] = src4[b, :, :L, :].transpose(1, 0, 2)
    return dst


# ---------------------------------------------------------------------------------------
# scale_mask_softmax  (scale_mask_softmax_kernel.cu:12-42)
# ---------------------------------------------------------------------------------------
def scale_mask_softmax(src, real_seq_len, batch_size, batch_seq_len, head_num):
    """In-place semantics of ker_scale_mask_softmax: for batch b, every query row
    i < real_seq_len[b] becomes softmax over keys j <= i (fp32 max / exp / sum), keys
    j > i become exactly 0; rows i >= real_seq_len[b] are left untouched.  No scale is
    applied.  Returns a new array of src's dtype."""
    S = batch_seq_len
    x = src.reshape(batch_size, head_num, S, S)
    out = x.copy()
    xf = x.astype(np.float32)
    causal = np.tril(np.ones((S, S), dtype=bool))
    masked = np.where(causal, xf, -np.inf)
    m = masked.max(axis=-1, keepdims=True)
    e = np.where(causal, np.exp(masked - m, dtype=np.float32), np.float32(0))
    p = (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(src.dtype)
    for b in range(batch_size):
        L = min(int(real_seq_len[b]), S)
        out[b, :, :L, :] = p[b, :, :L, :]
    return out.reshape(src.shape)


# ---------------------------------------------------------------------------------------
# fused LayerNorm forward  (layer_norm_cuda_kernel.cu:243-279)
# ---------------------------------------------------------------------------------------
def layer_norm_fwd(x, gamma, beta, eps, out_dtype=None):
    """cuApplyLayerNorm: per row, fp32 mean and biased variance (Welford in the kernel; a
    float64 two-pass sum here is the exact value it approximates), invvar = 1/sqrt(var+eps),
    y = gamma * (x - mean) * invvar + beta.  Returns (y, mean[n1] fp32, invvar[n1] fp32);
    y is evaluated in float64 and cast once to out_dtype (the kernel rounds twice in the
    output type, which stays inside the float tolerance of the tests)."""
    out_dtype = out_dtype or x.dtype
    n2 = x.shape[-1]
    x2 = x.reshape(-1, n2).astype(np.float64)
    mu = x2.mean(axis=1)
    var = ((x2 - mu[:, None]) ** 2).mean(axis=1)
    invvar = 1.0 / np.sqrt(var + eps)
    y = (x2 - mu[:, None]) * invvar[:, None]
    if gamma is not None:
        y = y * gamma.astype(np.float64)[None, :] + beta.astype(np.float64)[None, :]
    return y.astype(out_dtype).reshape(x.shape), mu.astype(np.float32), invvar.astype(np.float32)


# ---------------------------------------------------------------------------------------
# linear  (linear_wrapper.cpp:98-108)
# ---------------------------------------------------------------------------------------
def linear(x, w):
    """mlp_gemm: out[b, s, :] = x[b, s, :] @ w.T (no bias).  Evaluated in float64 and cast
    to x's dtype; the reference accumulates in fp16, which is strictly less accurate."""
    return (x.astype(np.float64) @ w.astype(np.float64).T).astype(x.dtype)
