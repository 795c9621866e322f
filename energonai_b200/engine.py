"""launch_engine / AsyncEngine with the reference's interface (energonai/engine.py:23-168): a
master that batches submitted requests, sends each batch to every tensor-parallel worker over
torch RPC and hands results back by request id.

Kept: constructor and method names, `submit` / `wait` / `get` / `shutdown`, QueueFullError, the
BatchManager hooks, "same batch to every rank, rank 0's answer is returned" (engine.py:79-80,
94-97).  Changed: one pipeline stage only (pp_world_size must be 1), blocking queues instead of
10 ms polling, workers stop through an RPC that sets an event instead of raising SIGINT."""
import asyncio
import threading
import time
from collections import deque
from typing import Any, Callable, Deque, Dict, Hashable, List, Optional

import torch.distributed.rpc as trpc
import torch.nn as nn

from .batch_mgr import BatchManager, SubmitEntry
from .pipe import Pipe
from .task import TaskEntry
from .worker import _request_stop, launch_workers, rpc_options


class QueueFullError(Exception):
    pass


class AsyncEngine:
    def __init__(self, tp_world_size: int, pp_world_size: int, master_host: str, rpc_port: int, n_proc_per_node: int,
                 batch_manager: Optional[BatchManager] = None, pipe_size: int = 1, queue_size: int = 0,
                 rpc_disable_shm: bool = True) -> None:
        if pp_world_size != 1:
            raise RuntimeError("pipeline parallelism is outside this package: pp_world_size must be 1")
        self.batch_manager = batch_manager if batch_manager is not None else BatchManager()
        assert isinstance(self.batch_manager, BatchManager)
        self.world_size = tp_world_size * pp_world_size
        trpc.init_rpc("master", rank=0, world_size=self.world_size + 1,
                      rpc_backend_options=rpc_options(master_host, rpc_port, rpc_disable_shm))
        self.completion_pipes: List[Pipe] = [Pipe(f"{i}_to_m", f"worker{i}", "master") for i in range(self.world_size)]
        for pipe in self.completion_pipes:
            assert pipe.recv() == 0                      # every worker reports pipeline rank 0
        self.submit_pipes: List[Pipe] = [Pipe(f"m_to_{i}", "master", f"worker{i}", max_size=pipe_size)
                                         for i in range(self.world_size)]
        self.queue_size = queue_size
        self.lock = threading.Lock()
        self.work = threading.Condition(self.lock)
        self.submit_queue: Deque[SubmitEntry] = deque()
        self.batch_info: Dict[Hashable, Any] = {}
        self.completion_map: Dict[Hashable, Any] = {}
        self.running = True
        self.submit_thread = threading.Thread(target=self._submit_loop, daemon=True)
        self.completion_thread = threading.Thread(target=self._completion_loop, daemon=True)
        self.submit_thread.start()
        self.completion_thread.start()

    def _submit_loop(self) -> None:
        while True:
            with self.work:
                while self.running and not self.submit_queue:
                    self.work.wait(0.1)
                if not self.running:
                    return
                task_entry, info = self.batch_manager.make_batch(self.submit_queue)
                self.batch_info[task_entry.uids] = (info, len(task_entry.uids), time.time())
            for pipe in self.submit_pipes:               # the same batch goes to every tensor-parallel rank
                pipe.send(task_entry)

    def _completion_loop(self) -> None:
        while self.running:
            try:
                first: TaskEntry = self.completion_pipes[0].recv(timeout=0.1)
            except RuntimeError:
                continue
            for pipe in self.completion_pipes[1:]:       # drain the other ranks' copies of the same batch
                while self.running:
                    try:
                        pipe.recv(timeout=0.1)
                        break
                    except RuntimeError:
                        continue
            with self.lock:
                info, _, _ = self.batch_info.pop(first.uids)
                for uid, output in self.batch_manager.split_batch(first, **info):
                    self.completion_map[uid] = output

    def submit(self, uid: Hashable, data: Any) -> None:
        assert self.submit_thread.is_alive()
        with self.work:
            assert uid not in self.completion_map
            if self.queue_size > 0 and len(self.submit_queue) >= self.queue_size:
                raise QueueFullError(f"Submit queue full, size: {self.queue_size}")
            self.submit_queue.append(SubmitEntry(uid, data))
            self.work.notify()

    def _take(self, uid: Hashable):
        with self.lock:
            if uid in self.completion_map:
                return True, self.completion_map.pop(uid)
        return False, None

    async def wait(self, uid: Hashable) -> Any:
        while True:
            done, out = self._take(uid)
            if done:
                return out
            await asyncio.sleep(0.005)

    def get(self, uid: Hashable, interval: float = 0.005) -> Any:
        while True:
            done, out = self._take(uid)
            if done:
                return out
            time.sleep(interval)

    def shutdown(self) -> None:
        with self.work:
            if not self.running:
                return
            self.running = False
            self.work.notify_all()
        for i in range(self.world_size):
            trpc.rpc_sync(f"worker{i}", _request_stop)
        trpc.shutdown()
        self.submit_thread.join()
        self.completion_thread.join()


def launch_engine(tp_world_size: int, pp_world_size: int, master_host: str, master_port: int, rpc_port: int,
                  model_fn: Callable[..., nn.Module], n_nodes: int = 1, node_rank: int = 0,
                  batch_manager: Optional[BatchManager] = None, pipe_size: int = 1, queue_size: int = 0,
                  rpc_disable_shm: bool = True, **model_kwargs: Any) -> Optional[AsyncEngine]:
    world_size = tp_world_size * pp_world_size
    assert world_size % n_nodes == 0
    n_proc_per_node = world_size // n_nodes
    launch_workers(tp_world_size, pp_world_size, master_host, master_port, rpc_port, model_fn,
                   n_proc_per_node=n_proc_per_node, node_rank=node_rank, pipe_size=pipe_size,
                   rpc_disable_shm=rpc_disable_shm, **model_kwargs)
    if node_rank == 0:
        return AsyncEngine(tp_world_size, pp_world_size, master_host, rpc_port, n_proc_per_node,
                           batch_manager=batch_manager, pipe_size=pipe_size, queue_size=queue_size,
                           rpc_disable_shm=rpc_disable_shm)
    return None
