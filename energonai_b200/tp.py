"""Tensor-parallel context: which rank of which group this process is, and the all-reduce the
row-parallel layers use.

The reference gets this from colossalai's global context (`gpc`, ParallelMode.PARALLEL_1D;
set up by colossalai.launch at energonai/worker.py:27-28).  Here it is a small explicit object
over torch.distributed: one process per GPU, NCCL over NVLink as the collective backend.
With no context installed every layer behaves as tensor-parallel size 1.
"""
import torch
import torch.distributed as dist


class TPContext:
    def __init__(self, group=None, rank=0, world_size=1):
        self.group, self.rank, self.world_size = group, rank, world_size
        self.peer = None       # PeerExchange for the fused GEMM + all-reduce (enable_peer_exchange)

    def enable_peer_exchange(self, max_rows, max_cols, bulk_rows=0):
        """Allocates and maps the NVLink exchange areas (collective over the group).  Row-parallel
        layers then carry their all-reduce in the library's own kernels: for up to max_rows
        (<= 128) x max_cols outputs inside the GEMM epilogue or the chained generation step, and,
        with bulk_rows > 0, for prompt-sized products of up to bulk_rows x max_cols as a
        reduce-scatter in the GEMM epilogue followed by a reduce-and-broadcast kernel.  Anything
        larger keeps using NCCL."""
        if self.world_size > 1 and self.peer is None:
            from .comm import PeerExchange
            self.peer = PeerExchange(self.group, self.rank, self.world_size, max_rows, max_cols, bulk_rows=bulk_rows)
        return self.peer

    def enable_peer_exchange_for(self, model, max_rows=128, bulk_rows=8192):
        """enable_peer_exchange sized for `model`: the widest row-parallel output it contains,
        and prompts of up to bulk_rows tokens per batch."""
        from .nn import Linear1D_Row
        cols = [m.out_features for m in model.modules() if isinstance(m, Linear1D_Row)]
        if self.world_size <= 1 or not cols:
            return None
        if self.world_size > 4:
            bulk_rows = 0      # among 8 ranks the prompt-sized exchange was measured erratic: NCCL carries prompts there
        return self.enable_peer_exchange(max_rows, max(cols), bulk_rows=bulk_rows)

    def all_reduce(self, t):
        """In-place SUM over the tensor-parallel group (no-op for one rank).  Small CUDA tensors go
        through the library's one-shot exchange over NVLink peer memory when it is enabled
        (latency-bound messages of generation steps); everything else through NCCL."""
        if self.world_size > 1:
            p = self.peer
            if (p is not None and t.is_cuda and t.is_contiguous() and t.dtype in _ONE_SHOT_DTYPES
                    and p.fits_bytes(t.numel() * t.element_size())):
                p.all_reduce(t)
            else:
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_gather_last_dim(self, t):
        if self.world_size == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


_ONE_SHOT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
_ctx = TPContext()


def get_tp():
    return _ctx


def set_tp(ctx):
    global _ctx
    _ctx = ctx if ctx is not None else TPContext()
    return _ctx


def init_tp(tp_world_size=None, group=None):
    """Installs a context over an initialised torch.distributed default group (or `group`)."""
    if not dist.is_initialized():
        return set_tp(TPContext())
    group = group if group is not None else dist.group.WORLD
    ws = dist.get_world_size(group)
    if tp_world_size is not None and tp_world_size != ws:
        raise RuntimeError(f"tensor-parallel size {tp_world_size} does not match the process group size {ws}")
    return set_tp(TPContext(group, dist.get_rank(group), ws))


def divide(numerator, denominator):
    if numerator % denominator != 0:
        raise ValueError(f"{numerator} is not divisible by {denominator}")
    return numerator // denominator
