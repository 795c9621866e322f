"""Python entry to eb_decode_chain: several dependent generation-step operations (small-batch
GEMMs and LayerNorms) in one persistent launch."""
import ctypes

import torch

from ._lib import lib, check, dtype_code, stream_ptr, require_cuda
from .gemm import ACT_CODES

OP_GEMM, OP_LAYERNORM, OP_REDUCE_LAYERNORM = 0, 1, 2
MAX_OPS = 8


class ChainOp(ctypes.Structure):
    """struct eb_chain_op of include/energon_b200.h, field for field."""
    _fields_ = [("type", ctypes.c_int),
                ("A", ctypes.c_void_p), ("lda", ctypes.c_longlong),
                ("W", ctypes.c_void_p), ("ldw", ctypes.c_longlong),
                ("C", ctypes.c_void_p), ("ldc", ctypes.c_longlong),
                ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("ldr", ctypes.c_longlong),
                ("N", ctypes.c_int), ("K", ctypes.c_int), ("out_dtype", ctypes.c_int), ("act", ctypes.c_int),
                ("c_rows_per_batch", ctypes.c_int), ("c_batch_stride", ctypes.c_longlong),
                ("c_row_offset_device", ctypes.c_void_p),
                ("c_row_offset_limit", ctypes.c_int), ("exchange", ctypes.c_int),
                ("x", ctypes.c_void_p), ("y", ctypes.c_void_p), ("gamma", ctypes.c_void_p), ("beta", ctypes.c_void_p),
                ("n2", ctypes.c_int), ("eps", ctypes.c_double)]


def _p(t):
    return None if t is None else t.data_ptr()


def gemm_op(a, w, out=None, bias=None, residual=None, act=None, out_rows_per_batch=0, out_batch_stride=0, out_ld=None,
            out_row_offset_device=None, out_row_limit=0, exchange=False):
    """C = act(a @ w.T + bias) + residual as one operation of a chain; arguments as gemm().
    exchange=True: `w` is this rank's column shard of a row-parallel layer; the product is sent
    to the ranks of the chain's context instead of being stored (no out, bias, residual or act)
    and the next operation must be reduce_layernorm_op()."""
    require_cuda(a, w, out, bias, residual, out_row_offset_device)
    if exchange:
        if out is not None or bias is not None or residual is not None or act not in (None, "none", 0):
            raise RuntimeError("chain gemm: an exchanged product takes no out, bias, residual or activation")
        op = ChainOp()
        op.type, op.exchange = OP_GEMM, 1
        op.A, op.lda, op.W, op.ldw = a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0)
        op.N, op.K = w.shape[0], w.shape[1]
        op.out_dtype = dtype_code(a.dtype)
        op._keep = (a, w)
        return op
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.stride(1) != 1 or w.stride(1) != 1:
        raise RuntimeError("chain gemm: a [M,K] and w [N,K] with contiguous rows required")
    if residual is not None and (residual.stride(-1) != 1 or residual.dtype != a.dtype):
        raise RuntimeError("chain gemm: residual must be row-major and of the operand dtype")
    op = ChainOp()
    op.type = OP_GEMM
    op.A, op.lda, op.W, op.ldw = a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0)
    op.C, op.ldc = out.data_ptr(), (out_ld if out_ld is not None else out.stride(0))
    op.bias, op.residual = _p(bias), _p(residual)
    op.ldr = residual.stride(0) if residual is not None else 0
    op.N, op.K = w.shape[0], w.shape[1]
    op.out_dtype = dtype_code(out.dtype)
    op.act = ACT_CODES[act] if not isinstance(act, int) else act
    op.c_rows_per_batch, op.c_batch_stride = out_rows_per_batch, out_batch_stride
    op.c_row_offset_device = _p(out_row_offset_device)
    op.c_row_offset_limit = int(out_row_limit)
    op._keep = (a, w, out, bias, residual, out_row_offset_device)
    return op


def layernorm_op(x, y, gamma, beta, eps):
    """y = gamma * (x - mean) / sqrt(var + eps) + beta over the rows of x [M, n2]."""
    require_cuda(x, y, gamma, beta)
    if x.dim() != 2 or not x.is_contiguous() or not y.is_contiguous() or x.shape != y.shape:
        raise RuntimeError("chain layernorm: contiguous x and y of one shape [M, n2] required")
    op = ChainOp()
    op.type = OP_LAYERNORM
    op.x, op.y, op.gamma, op.beta = x.data_ptr(), y.data_ptr(), gamma.data_ptr(), beta.data_ptr()
    op.n2, op.eps = x.shape[1], float(eps)
    op._keep = (x, y, gamma, beta)
    return op


def reduce_layernorm_op(sum_out, n_cols, bias=None, residual=None, y=None, gamma=None, beta=None, eps=1e-5):
    """sum_out = (sum over ranks of the preceding exchanged product) + bias + residual, then
    y = LayerNorm(sum_out; gamma, beta) (skipped when gamma is None).  sum_out / residual / y are
    [M, n_cols] row-major."""
    require_cuda(sum_out, bias, residual, y, gamma, beta)
    if sum_out.dim() != 2 or sum_out.stride(1) != 1 or sum_out.shape[1] != n_cols:
        raise RuntimeError("chain reduce: sum_out must be [M, n_cols] with contiguous rows")
    if gamma is not None and (y is None or beta is None or not y.is_contiguous()):
        raise RuntimeError("chain reduce: gamma needs beta and a contiguous y")
    op = ChainOp()
    op.type = OP_REDUCE_LAYERNORM
    op.C, op.ldc = sum_out.data_ptr(), sum_out.stride(0)
    op.bias, op.residual = _p(bias), _p(residual)
    op.ldr = residual.stride(0) if residual is not None else 0
    op.y, op.gamma, op.beta = _p(y), _p(gamma), _p(beta)
    op.n2, op.eps = int(n_cols), float(eps)
    op._keep = (sum_out, bias, residual, y, gamma, beta)
    return op


class Chain:
    """A fixed sequence of operations over fixed buffers, launched with run().  Needs a
    zero-filled workspace (arrival counters, stream-K partial sums): its own, or one passed in."""

    @staticmethod
    def workspace_bytes(ops, M, device):
        arr = (ChainOp * len(ops))(*ops)
        with torch.cuda.device(device):
            return lib().eb_decode_chain_workspace_bytes(ctypes.cast(arr, ctypes.c_void_p), len(ops), int(M))

    def __init__(self, ops, M, dtype, device, workspace=None, comm=None):
        if not 1 <= len(ops) <= MAX_OPS:
            raise RuntimeError(f"chain: 1..{MAX_OPS} operations")
        self.ops = (ChainOp * len(ops))(*ops)
        self._keep = [o._keep for o in ops]
        self.n, self.M, self.dtype = len(ops), int(M), dtype_code(dtype)
        self.comm = comm                 # PeerExchange of the tensor-parallel group, for exchanged products
        with torch.cuda.device(device):
            nbytes = lib().eb_decode_chain_workspace_bytes(ctypes.cast(self.ops, ctypes.c_void_p), self.n, self.M)
        if nbytes == 0:
            raise RuntimeError("chain: unsupported shape (M must be in [1, 128])")
        self.nbytes = nbytes
        if workspace is not None and workspace.numel() < nbytes:
            raise RuntimeError(f"chain: the shared workspace holds {workspace.numel()} bytes, {nbytes} needed")
        # a workspace may be shared by chains that never overlap on the device (one stream)
        self.ws = workspace if workspace is not None else torch.zeros(nbytes, dtype=torch.uint8, device=device)

    def run(self):
        check(lib().eb_decode_chain(ctypes.cast(self.ops, ctypes.c_void_p), self.n, self.M, self.dtype, self.ws.data_ptr(),
                                    self.ws.numel(), self.comm.handle if self.comm is not None else None, stream_ptr()),
              "decode_chain")
