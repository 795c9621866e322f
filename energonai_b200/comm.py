"""Peer-addressable exchange areas for the fused row-parallel GEMM + all-reduce.

One `PeerExchange` per tensor-parallel group and process: a receive area and a flag area
allocated as symmetric memory (every rank allocates the same sizes, the handles are exchanged
through the process group, and each rank maps its peers' areas over NVLink).  torch's
symmetric-memory allocator is used only for that plumbing; the data movement is done by the
GEMM kernel's own peer stores (eb_gemm_allreduce).

The reference reaches the same result with a blocking NCCL all-reduce inside colossalai's
Linear1D_Row (used at energonai/model/attention.py:37, energonai/model/mlp.py:22).
"""
import ctypes

import torch
import torch.distributed as dist

FLAG_SLOTS = 1024          # tiles of 128 output columns per (parity, source): N up to 131072


class PeerExchange:
    def __init__(self, group, rank, world, max_rows, max_cols):
        import torch.distributed._symmetric_memory as symm_mem
        from ._lib import lib
        self.rank, self.world = rank, world
        self.max_rows, self.max_cols = max_rows, max_cols
        self.recv_bytes = lib().eb_gemm_allreduce_recv_bytes(world, max_rows, max_cols)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.recv = symm_mem.empty(max(self.recv_bytes // 4, 4), dtype=torch.float32, device=dev)
        self.flags = symm_mem.empty(2 * world * FLAG_SLOTS, dtype=torch.int32, device=dev)
        self.recv.zero_()
        self.flags.zero_()
        self._h_recv = symm_mem.rendezvous(self.recv, group)
        self._h_flags = symm_mem.rendezvous(self.flags, group)
        PtrArray = ctypes.c_void_p * world
        self.recv_ptrs = PtrArray(*[int(p) for p in self._h_recv.buffer_ptrs])
        self.flag_ptrs = PtrArray(*[int(p) for p in self._h_flags.buffer_ptrs])
        self.calls = 0
        torch.cuda.synchronize()
        dist.barrier(group=group)          # nobody sends before every area is zeroed and mapped

    def fits(self, rows, cols):
        from ._lib import lib
        need = lib().eb_gemm_allreduce_recv_bytes(self.world, rows, cols)
        return 0 < rows <= 128 and 0 < need <= self.recv_bytes and (cols + 127) // 128 <= FLAG_SLOTS

    def next_parity(self):
        p = self.calls & 1
        self.calls += 1
        return p
