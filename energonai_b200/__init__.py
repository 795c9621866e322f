"""energonai_b200: EnergonAI's tensor-parallel transformer layer forward for B200 (sm_100a).

`energonai_b200.kernel` mirrors `energonai.kernel`; `energonai_b200.model` mirrors the layer
modules of `energonai.model`.  All compute runs in hand-written CUDA behind the C ABI
declared in include/energon_b200.h; there is no CPU or PyTorch fallback.
"""
__version__ = "0.1.0"

from .batch_mgr import BatchManager, BatchManagerForGeneration, SubmitEntry
from .task import TaskEntry


def __getattr__(name):
    # launch_engine and QueueFullError pull in torch.distributed.rpc; import them on first use
    if name in ("launch_engine", "QueueFullError", "AsyncEngine", "WorkerFailedError"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)


__all__ = ["BatchManager", "BatchManagerForGeneration", "launch_engine", "SubmitEntry", "TaskEntry", "QueueFullError",
           "WorkerFailedError"]
