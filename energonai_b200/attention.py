"""Python entry to the fused attention kernels (eb_attention_prefill[_tc] / eb_attention_decode)."""
import os

import torch

from ._lib import lib, check, dtype_code, ptr, stream_ptr, require_cuda

_scratch = {}
TC_MIN_ROWS = 128        # below this many query rows the 256-row CTAs of the tensor-core kernel are mostly padding


def _get_scratch(device, nbytes):
    key = torch.device(device).index
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _bsh_strides(t, head_dim):
    """(batch_stride, row_stride) of a [B, S, H*D] view whose last dim is contiguous."""
    if t.dim() != 3 or t.stride(2) != 1 or t.shape[2] % head_dim:
        raise RuntimeError("attention: tensors must be [batch, seq, heads*head_dim] views with a contiguous last dim")
    return t.stride(0), t.stride(1)


def attention_prefill(q, k, v, head_dim, mask=None, causal=True, scale=None, out=None, impl=None):
    """q [B,Sq,H*D], k/v [B,Sk,H*D] (strided views allowed), mask [B,Sk] additive or None.
    Returns out [B,Sq,H*D].  impl: "tc" (tcgen05 kernel), "mma" (mma.sync kernel) or None =
    "tc" for prompts of at least TC_MIN_ROWS rows (EB_ATTN_TC=0 keeps "mma")."""
    require_cuda(q, k, v, mask, out)
    B, Sq, HD = q.shape
    Sk = k.shape[1]
    H = HD // head_dim
    if out is None:
        out = torch.empty((B, Sq, HD), dtype=q.dtype, device=q.device)
    if mask is not None:
        if mask.dtype != q.dtype or mask.stride(-1) != 1 or mask.dim() != 2 or mask.shape[1] < Sk:
            raise RuntimeError("attention: mask must be [batch, kv_len] of the tensor dtype")
    qs, ks, vs, os_ = (_bsh_strides(t, head_dim) for t in (q, k, v, out))
    scale = head_dim ** -0.5 if scale is None else scale
    if impl is None:
        impl = "tc" if Sq >= TC_MIN_ROWS and os.environ.get("EB_ATTN_TC", "1") != "0" else "mma"
    if impl == "tc":
        check(lib().eb_attention_prefill_tc(ptr(q), ptr(k), ptr(v), ptr(out), ptr(mask), qs[0], qs[1], ks[0], ks[1], vs[0],
                                            vs[1], os_[0], os_[1], mask.stride(0) if mask is not None else 0, B, H, Sq, Sk,
                                            head_dim, 1 if causal else 0, float(scale), dtype_code(q.dtype), stream_ptr()),
              "attention_prefill_tc")
        return out
    check(lib().eb_attention_prefill(ptr(q), ptr(k), ptr(v), ptr(out), ptr(mask), qs[0], qs[1], ks[0], ks[1], vs[0], vs[1],
                                     os_[0], os_[1], mask.stride(0) if mask is not None else 0, B, H, Sq, Sk, head_dim,
                                     1 if causal else 0, float(scale), dtype_code(q.dtype), stream_ptr()),
          "attention_prefill")
    return out


def pick_nsplit(batch, heads, kv_len, sm_count=148):
    """Key splits per (sequence, head).  Splitting costs a merge and shortens every CTA's stream,
    and was measured to lose whenever a CTA would be left with fewer than about a thousand keys:
    at 576 keys and batch 16, 1 / 2 / 3 / 6 splits take 30.9 / 34.7 / 36.2 / 41.3 us per layer with
    40 heads and 7.9 / 9.1 / 9.7 / 10.0 us with the 5 heads of an 8-way shard (80 CTAs on 148 SMs:
    even an underfilled machine prefers whole streams).  So: one split per 1024 keys, never more
    than gives every SM its three resident CTAs, never more than one per 64-key tile."""
    tiles = max(1, (kv_len + 63) // 64)
    want = -(-3 * sm_count // max(1, batch * heads))
    return max(1, min(want, kv_len // 1024, tiles, 64))


def attention_decode(q, k, v, head_dim, kv_len, mask=None, scale=None, out=None, nsplit=None, kv_len_device=None,
                     q_in_cache=False):
    """q [B, H*D] (one row per sequence), k/v [B, >=kv_len, H*D] cache views, mask [B, >=kv_len].
    With q_in_cache, q is a [B, capacity, H*D] view like k/v and the query is its row kv_len-1.
    Returns out [B, H*D]."""
    require_cuda(q, k, v, mask, out, kv_len_device)
    q_rs = 0
    if q_in_cache:
        q_rs = q.stride(1)
        q = q[:, 0]
    B, HD = q.shape
    H = HD // head_dim
    if q.stride(1) != 1:
        raise RuntimeError("attention_decode: q rows must be contiguous")
    if out is None:
        out = torch.empty((B, HD), dtype=q.dtype, device=q.device)
    ks, vs = _bsh_strides(k, head_dim), _bsh_strides(v, head_dim)
    if mask is not None and (mask.dtype != q.dtype or mask.stride(-1) != 1 or mask.dim() != 2):
        raise RuntimeError("attention: mask must be [batch, kv_len] of the tensor dtype")
    if nsplit is None:
        nsplit = pick_nsplit(B, H, kv_len)
    nbytes = lib().eb_attention_decode_scratch_bytes(B, H, head_dim, nsplit)
    scratch = _get_scratch(q.device, nbytes) if nbytes else None
    scale = head_dim ** -0.5 if scale is None else scale
    check(lib().eb_attention_decode(ptr(q), ptr(k), ptr(v), ptr(out), ptr(mask), q.stride(0), q_rs, ks[0], ks[1], vs[0], vs[1],
                                    out.stride(0), mask.stride(0) if mask is not None else 0, B, H, int(kv_len),
                                    ptr(kv_len_device), head_dim, float(scale), dtype_code(q.dtype), nsplit, ptr(scratch),
                                    scratch.numel() if scratch is not None else 0, stream_ptr()), "attention_decode")
    return out
