"""Python entry to the tcgen05 GEMM (eb_gemm): C = act(A @ W.T + bias) + residual."""
import torch

from ._lib import lib, check, dtype_code, ptr, stream_ptr, require_cuda, ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_GELU_ERF

ACT_CODES = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "gelu_tanh": ACT_GELU_TANH, "gelu": ACT_GELU_ERF}

_workspaces = {}


def workspace(device, nbytes):
    """Per-device scratch for the small-M (generation-step) GEMM: zero-filled once, grown on
    demand.  One buffer per device is enough because calls on a device are issued on one stream."""
    key = torch.device(device).index
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def gemm(a, w, bias=None, act=None, residual=None, out=None, out_dtype=None, out_rows_per_batch=0,
         out_batch_stride=0, out_ld=None, out_row_offset_device=None, out_row_limit=0, static_weight=False, peer=None,
         ln_fold=None):
    """a [M,K] (row stride allowed), w [N,K]; returns out [M,N].

    `out`, if given, receives the result; with out_rows_per_batch > 0 row m is written at
    element (m // rpb) * out_batch_stride + (m % rpb) * out_ld of `out` (a view into a cache);
    out_row_offset_device (int32 device scalar) adds that many rows of out_ld at run time;
    out_row_limit > 0 is the number of rows that offset may address (beyond it the kernel
    stores nothing and raises the device status word).
    static_weight=True promises that `w` is not being written by earlier work still in flight
    on the stream (model weights), which lets the kernel prefetch it early.
    ln_fold=(colsum, bias32, eps), from fold_layernorm(): `a` is the un-normalised input of a
    LayerNorm and `w` the weight with the LayerNorm scale folded in (M <= 32 only).
    (Asking a launch to pull the NEXT launch's weights into L2 was tried and removed: measured on
    B200 it slowed the generation step at every size, 6.50 -> 6.70 / 7.28 ms for 16 / 64 MB on one
    GPU and 2.50 -> 2.57 / 2.63 ms on an 8-way shard.)"""
    require_cuda(a, w, bias, residual, out)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise RuntimeError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T do not match")
    if a.dtype != w.dtype or a.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("gemm: fp16 or bf16 operands of one dtype required")
    if a.stride(1) != 1:
        a = a.contiguous()
    if w.stride(1) != 1:
        w = w.contiguous()
    M, K = a.shape
    N = w.shape[0]
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out_ld is None:
        out_ld = out.stride(0) if out.dim() == 2 else N
    if residual is not None and (residual.stride(-1) != 1 or residual.dtype != a.dtype):
        raise RuntimeError("gemm: residual must be row-major and of the operand dtype")
    code = ACT_CODES[act] if not isinstance(act, int) else act
    nbytes = lib().eb_gemm_workspace_bytes(M, N, K)
    ws = workspace(a.device, nbytes) if nbytes else None
    if ln_fold is not None:
        colsum, bias32, eps = ln_fold
        if bias is not None or peer is not None:
            raise RuntimeError("gemm: ln_fold carries the bias and does not combine with the peer exchange")
        if colsum.dtype != torch.float32 or bias32.dtype != torch.float32 or colsum.numel() != N or bias32.numel() != N:
            raise RuntimeError("gemm: ln_fold vectors must be fp32 of length N")
        check(lib().eb_gemm_ln(ptr(a), a.stride(0), ptr(w), w.stride(0), ptr(out), out_ld, ptr(colsum), ptr(bias32), float(eps),
                               ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K,
                               dtype_code(a.dtype), dtype_code(out_dtype), code, out_rows_per_batch, out_batch_stride,
                               ptr(out_row_offset_device), int(out_row_limit), 1 if static_weight else 0, ptr(ws),
                               ws.numel() if ws is not None else 0, stream_ptr()), "gemm_ln")
        return out
    if peer is not None:
        if not peer.fits(M, N):
            raise RuntimeError(f"gemm: {M} x {N} does not fit the peer exchange areas")
        check(lib().eb_gemm_allreduce(ptr(a), a.stride(0), ptr(w), w.stride(0), ptr(out), out_ld, ptr(bias), ptr(residual),
                                      residual.stride(0) if residual is not None else 0, M, N, K, dtype_code(a.dtype),
                                      dtype_code(out_dtype), code, out_rows_per_batch, out_batch_stride,
                                      ptr(out_row_offset_device), int(out_row_limit), 1 if static_weight else 0, ptr(ws),
                                      ws.numel() if ws is not None else 0, peer.handle, stream_ptr()),
              "gemm_allreduce")
        return out
    check(lib().eb_gemm(ptr(a), a.stride(0), ptr(w), w.stride(0), ptr(out), out_ld, ptr(bias), ptr(residual),
                        residual.stride(0) if residual is not None else 0, M, N, K, dtype_code(a.dtype),
                        dtype_code(out_dtype), code, out_rows_per_batch, out_batch_stride,
                        ptr(out_row_offset_device), int(out_row_limit), 1 if static_weight else 0, ptr(ws),
                        ws.numel() if ws is not None else 0, stream_ptr()), "gemm")
    return out


LN_FOLD_MAX_ROWS = 32


def fold_layernorm(weight, bias, gamma, beta):
    """One-time preparation for gemm(..., ln_fold=...): y = LayerNorm(x; gamma, beta) @ weight.T + bias
    equals rstd * (x @ w_folded.T - mean * colsum) + bias32 with
      w_folded = weight * gamma (rounded to the weight dtype), colsum = w_folded.sum(1),
      bias32 = bias + weight @ beta   (fp32).
    Returns (w_folded, colsum, bias32)."""
    with torch.no_grad():
        w32 = weight.detach().float()
        w_folded = (w32 * gamma.detach().float()[None, :]).to(weight.dtype).contiguous()
        colsum = w_folded.float().sum(1).contiguous()
        bias32 = w32 @ beta.detach().float()
        if bias is not None:
            bias32 = bias32 + bias.detach().float()
        return w_folded, colsum, bias32.contiguous()


def device_status(clear=True):
    """(code, where, block, detail) of the current device's bounded-wait status word."""
    import ctypes
    buf = (ctypes.c_int * 4)()
    check(lib().eb_device_status(ctypes.cast(buf, ctypes.c_void_p), 1 if clear else 0), "device_status", launches=0)
    return tuple(buf)
