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


class PeerExchange:
    """One eb_comm.  `max_rows` x `max_cols` (16-bit elements) is the largest partial product one
    exchange carries; rows are rounded up the way the generation-step GEMM pads its batch."""

    def __init__(self, group, rank, world, max_rows, max_cols, wait_budget_s=None):
        from ._lib import lib, check
        self.rank, self.world, self.group = rank, world, group
        self.max_rows, self.max_cols = max_rows, max_cols
        L = lib()
        half = L.eb_comm_exchange_bytes(world, self._padded(max_rows), max_cols)
        self.recv_bytes = 2 * ((half + 511) // 512 * 512)
        handle = ctypes.c_void_p()
        check(L.eb_comm_create(rank, world, self.recv_bytes, None, ctypes.byref(handle)), "comm_create", launches=0)
        self.handle = handle
        self._destroyed = False
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
    def from_pointers(cls, rank, world, recv_local, peer_ptrs, wait_budget_s=None):
        """A context over receive areas the caller allocated and mapped itself (one process
        driving several GPUs with peer access, or another symmetric allocator): `recv_local` is
        this rank's area (a zero-filled CUDA uint8 tensor, kept alive by the object), `peer_ptrs`
        the device addresses of all ranks' areas as seen from this process."""
        from ._lib import lib, check
        self = cls.__new__(cls)
        self.rank, self.world, self.group = rank, world, None
        self.max_rows = self.max_cols = None
        self.recv_bytes = recv_local.numel()
        self._area = recv_local
        handle = ctypes.c_void_p()
        check(lib().eb_comm_create(rank, world, self.recv_bytes, recv_local.data_ptr(), ctypes.byref(handle)), "comm_create",
              launches=0)
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
        return lib().eb_comm_exchange_bytes(self.world, self._padded(rows), cols) <= self.recv_bytes // 2

    def set_wait_budget(self, seconds):
        from ._lib import lib, check
        check(lib().eb_comm_set_wait_budget(self.handle, float(seconds)), "comm_set_wait_budget", launches=0)

    def status(self, clear=True):
        """(code, where, block, detail) of this context's own kernels (eb_allreduce)."""
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
        return self.world * nbytes * 2 <= self.recv_bytes // 2 and nbytes % 8 == 0

    def destroy(self):
        if not self._destroyed:
            from ._lib import lib
            lib().eb_comm_destroy(self.handle)
            self._destroyed = True
