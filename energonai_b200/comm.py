"""The tensor-parallel exchange context of the library (eb_comm_*) for one rank of a
torch.distributed group.

The library owns the context: it allocates this rank's receive area, exports a handle, maps the
peers' areas (CUDA IPC over NVLink) and keeps the sequence number of the exchanges in device
memory.  This module only carries the handles between the processes (one all_gather on the
caller's process group) and holds the opaque pointer.  The data movement is done by the
library's own kernels: the fused row-parallel GEMM + all-reduce (eb_gemm_allreduce), the
generation-step chain (eb_decode_chain) and the stand-alone one-shot all-reduce (eb_allreduce).

The reference reaches the same result with a blocking NCCL all-reduce inside colossalai's
Linear1D_Row (used at energonai/model/attention.py:37, energonai/model/mlp.py:22), on process
groups created by colossalai.launch (energonai/worker.py:27-28).
"""
import ctypes

import torch
import torch.distributed as dist


class _DevicePointer:
    """Lets torch wrap a raw device address (a slice of the context's bulk region)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerExchange:
    """One eb_comm.  `max_rows` x `max_cols` (16-bit elements) is the largest partial product a
    generation-step exchange carries (rows are rounded up the way the generation-step GEMM pads
    its batch); `bulk_rows` > 0 adds a bulk region for all-reducing prompt-sized products of up
    to bulk_rows x max_cols (one staging area and two alternating gather areas)."""

    def __init__(self, group, rank, world, max_rows, max_cols, bulk_rows=0, wait_budget_s=None):
        from ._lib import lib, check
        self.rank, self.world, self.group = rank, world, group
        self.max_rows, self.max_cols = max_rows, max_cols
        L = lib()
        half = L.eb_comm_exchange_bytes(world, self._padded(max_rows), max_cols)
        self.line_bytes = 2 * ((half + 511) // 512 * 512)
        self.bulk_bytes = 0
        if bulk_rows > 0:
            stage = L.eb_reduce_broadcast_stage_bytes(world, bulk_rows, max_cols)
            self.bulk_bytes = 3 * ((stage + 511) // 512 * 512)
        handle = ctypes.c_void_p()
        check(L.eb_comm_create(rank, world, self.line_bytes, self.bulk_bytes, None, ctypes.byref(handle)), "comm_create",
              launches=0)
        self.handle = handle
        self._destroyed = False
        self._gather_toggle = 0
        if world > 1:
            n = L.eb_comm_handle_bytes()
            blob = (ctypes.c_ubyte * n)()
            check(L.eb_comm_export_handle(self.handle, blob, n), "comm_export_handle", launches=0)
            mine = torch.tensor(list(bytes(blob)), dtype=torch.uint8)
            if dist.get_backend(group) == "nccl":
                mine = mine.cuda()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
            blobs = bytes(torch.cat([p.cpu() for p in parts]).tolist())
            if len(blobs) != world * n:
                raise RuntimeError("comm: truncated handle exchange")
            check(L.eb_comm_connect(self.handle, blobs, len(blobs)), "comm_connect", launches=0)
            torch.cuda.synchronize()
            dist.barrier(group=group)          # nobody sends before every area is zeroed and mapped
        if wait_budget_s is not None:
            self.set_wait_budget(wait_budget_s)

    @classmethod
    def from_pointers(cls, rank, world, recv_local, peer_ptrs, line_bytes=None, wait_budget_s=None):
        """A context over receive areas the caller allocated and mapped itself (one process
        driving several GPUs with peer access, or another symmetric allocator): `recv_local` is
        this rank's area (a zero-filled CUDA uint8 tensor, kept alive by the object), `peer_ptrs`
        the device addresses of all ranks' areas as seen from this process.  The area is 4096
        bytes of signal words, `line_bytes` of flagged lines (default: all the rest) and the
        bulk region behind them."""
        from ._lib import lib, check
        self = cls.__new__(cls)
        self.rank, self.world, self.group = rank, world, None
        self.max_rows = self.max_cols = None
        total = recv_local.numel()
        self.line_bytes = (total - 4096) // 512 * 512 if line_bytes is None else line_bytes
        self.bulk_bytes = (total - 4096 - self.line_bytes) // 512 * 512
        self._area = recv_local
        self._gather_toggle = 0
        handle = ctypes.c_void_p()
        check(lib().eb_comm_create(rank, world, self.line_bytes, self.bulk_bytes, recv_local.data_ptr(), ctypes.byref(handle)),
              "comm_create", launches=0)
        self.handle, self._destroyed = handle, False
        table = (ctypes.c_void_p * world)(*[int(p) for p in peer_ptrs])
        check(lib().eb_comm_connect_pointers(self.handle, table), "comm_connect_pointers", launches=0)
        if wait_budget_s is not None:
            self.set_wait_budget(wait_budget_s)
        return self

    @staticmethod
    def _padded(rows):
        return 16 if rows <= 16 else 32 if rows <= 32 else 64 if rows <= 64 else 128

    def fits(self, rows, cols):
        from ._lib import lib
        if not 0 < rows <= 128 or cols % 4:
            return False
        return lib().eb_comm_exchange_bytes(self.world, self._padded(rows), cols) <= self.line_bytes // 2

    def set_wait_budget(self, seconds):
        from ._lib import lib, check
        check(lib().eb_comm_set_wait_budget(self.handle, float(seconds)), "comm_set_wait_budget", launches=0)

    def status(self, clear=True):
        """(code, where, block, detail) of this context's own kernels (eb_allreduce, eb_reduce_broadcast)."""
        from ._lib import lib, check
        buf = (ctypes.c_int * 4)()
        check(lib().eb_comm_status(self.handle, buf, 1 if clear else 0), "comm_status", launches=0)
        return tuple(buf)

    def all_reduce(self, t):
        """In-place SUM of a contiguous CUDA tensor over the group with the library's one-shot
        kernel (small messages; fp32 / fp16 / bf16)."""
        from ._lib import lib, check, dtype_code, stream_ptr
        if not t.is_cuda or not t.is_contiguous():
            raise RuntimeError("comm.all_reduce: contiguous CUDA tensor required")
        check(lib().eb_allreduce(self.handle, t.data_ptr(), t.numel(), dtype_code(t.dtype), stream_ptr()), "allreduce")
        return t

    def fits_bytes(self, nbytes):
        return self.world * nbytes * 2 <= self.line_bytes // 2 and nbytes % 8 == 0

    # ---- prompt-sized products: reduce-scatter inside the GEMM, then reduce + broadcast ----
    def _bulk_layout(self, rows, cols):
        """(stage_offset, stage_bytes, gather_bytes) or None when [rows, cols] does not fit."""
        from ._lib import lib
        stage = lib().eb_reduce_broadcast_stage_bytes(self.world, rows, cols)
        stage_r = (stage + 511) // 512 * 512
        gather_r = (rows * cols * 2 + 511) // 512 * 512
        if rows <= 128 or cols % 8 or stage_r + 2 * gather_r > self.bulk_bytes:
            return None
        return 0, stage_r, gather_r

    def fits_bulk(self, rows, cols):
        return self._bulk_layout(rows, cols) is not None

    def bulk_view(self, offset, rows, cols, dtype):
        from ._lib import lib, check
        ptr, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().eb_comm_local_area(self.handle, ctypes.byref(ptr), ctypes.byref(nbytes)), "comm_local_area", launches=0)
        typestr = "<f2" if dtype == torch.float16 else "<i2"
        t = torch.as_tensor(_DevicePointer(ptr.value + offset, (rows, cols), typestr), device="cuda")
        return t if dtype == torch.float16 else t.view(dtype)

    def row_parallel(self, a, w, bias=None, residual=None):
        """sum over ranks of a @ w.T, + bias + residual, for a prompt-sized a [M > 128, K]: returns
        a [M, N] tensor that LIVES IN THE CONTEXT'S BULK REGION and is overwritten by the call
        after the next one (two gather areas alternate); callers consume it before that."""
        from ._lib import lib, check, dtype_code, ptr, stream_ptr
        M, K = a.shape
        N = w.shape[0]
        lay = self._bulk_layout(M, N)
        if lay is None:
            raise RuntimeError(f"comm.row_parallel: {M} x {N} does not fit the bulk region")
        stage_off, stage_b, gather_b = lay
        gather_off = stage_b + self._gather_toggle * gather_b
        self._gather_toggle ^= 1
        if a.stride(1) != 1:
            a = a.contiguous()
        check(lib().eb_gemm_reduce_scatter(ptr(a), a.stride(0), ptr(w), w.stride(0), M, N, K, dtype_code(a.dtype), 1,
                                           self.handle, stage_off, stream_ptr()), "gemm_reduce_scatter")
        check(lib().eb_reduce_broadcast(self.handle, M, N, dtype_code(a.dtype), stage_off, gather_off, ptr(bias), ptr(residual),
                                        residual.stride(0) if residual is not None else 0, stream_ptr()), "reduce_broadcast")
        return self.bulk_view(gather_off, M, N, a.dtype)

    def destroy(self):
        if not self._destroyed:
            from ._lib import lib
            lib().eb_comm_destroy(self.handle)
            self._destroyed = True
