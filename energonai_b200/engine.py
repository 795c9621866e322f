"""launch_engine / AsyncEngine with the reference's interface (energonai/engine.py:23-168): a
master that batches submitted requests, sends each batch to every tensor-parallel worker over
torch RPC and hands results back by request id.

Kept: constructor and method names, `submit` / `wait` / `get` / `shutdown`, QueueFullError, the
BatchManager hooks, "same batch to every rank, rank 0's answer is returned" (engine.py:79-80,
94-97).  Changed: one pipeline stage only (pp_world_size must be 1), blocking queues instead of
10 ms polling, workers stop through an RPC that sets an event instead of raising SIGINT.
Added (the reference waits forever in both cases): a batch whose model call raised is answered
with that error (`RemoteFailure` -> RuntimeError from `get` / `wait`, the worker keeps serving),
and a worker process that exits while the engine runs makes every pending and later `get` /
`wait` raise WorkerFailedError; `shutdown` then tears the RPC layer down without waiting for
the dead peer."""
import asyncio
import threading
import time
from collections import deque
from typing import Any, Callable, Deque, Dict, Hashable, List, Optional

import torch.distributed.rpc as trpc
import torch.nn as nn

from .batch_mgr import BatchManager, SubmitEntry
from .pipe import Pipe
from .task import RemoteFailure, TaskEntry
from .worker import _request_stop, launch_workers, rpc_options


class QueueFullError(Exception):
    pass


class WorkerFailedError(RuntimeError):
    """A worker process exited (or became unreachable) while the engine was running."""


class AsyncEngine:
    def __init__(self, tp_world_size: int, pp_world_size: int, master_host: str, rpc_port: int, n_proc_per_node: int,
                 batch_manager: Optional[BatchManager] = None, pipe_size: int = 1, queue_size: int = 0,
                 rpc_disable_shm: bool = True, worker_procs=()) -> None:
        if pp_world_size != 1:
            raise RuntimeError("pipeline parallelism is outside this package: pp_world_size must be 1")
        self.batch_manager = batch_manager if batch_manager is not None else BatchManager()
        assert isinstance(self.batch_manager, BatchManager)
        self.world_size = tp_world_size * pp_world_size
        self.worker_procs = list(worker_procs)          # local worker processes, watched for exits
        self._start_rpc(master_host, rpc_port, rpc_disable_shm)
        self.completion_pipes: List[Pipe] = [Pipe(f"{i}_to_m", f"worker{i}", "master") for i in range(self.world_size)]
        for rank, pipe in enumerate(self.completion_pipes):
            hello = self._recv_hello(rank, pipe)
            if isinstance(hello, RemoteFailure):         # the worker could not build its model shard
                self._abandon_rpc()
                raise WorkerFailedError(f"worker {hello.rank} failed to start: {hello.message}")
            assert hello == 0                            # every worker reports pipeline rank 0
        self.submit_pipes: List[Pipe] = [Pipe(f"m_to_{i}", "master", f"worker{i}", max_size=pipe_size)
                                         for i in range(self.world_size)]
        self.queue_size = queue_size
        self.lock = threading.Lock()
        self.work = threading.Condition(self.lock)
        self.submit_queue: Deque[SubmitEntry] = deque()
        self.batch_info: Dict[Hashable, Any] = {}
        self.completion_map: Dict[Hashable, Any] = {}
        self.running = True
        self.failed: Optional[str] = None
        self.submit_thread = threading.Thread(target=self._submit_loop, daemon=True)
        self.completion_thread = threading.Thread(target=self._completion_loop, daemon=True)
        self.submit_thread.start()
        self.completion_thread.start()

    # -- start-up: a worker that dies before it joins (model_fn raised before the RPC layer was
    # up, the process group could not form, the process was killed) must not hang the caller --
    def _dead_worker(self) -> Optional[str]:
        for rank, proc in enumerate(self.worker_procs):
            if proc.exitcode is not None:
                return f"worker process {rank} exited with code {proc.exitcode} during start-up"
        return None

    def _start_rpc(self, master_host: str, rpc_port: int, rpc_disable_shm: bool) -> None:
        """init_rpc waits for every peer; it runs in a helper thread while this one watches the
        worker processes, so a worker that never arrives ends the wait with an error."""
        result: Dict[str, Any] = {}

        def join() -> None:
            try:
                trpc.init_rpc("master", rank=0, world_size=self.world_size + 1,
                              rpc_backend_options=rpc_options(master_host, rpc_port, rpc_disable_shm))
                result["ok"] = True
            except Exception as exc:                     # noqa: BLE001 (reported to the caller below)
                result["error"] = exc

        t = threading.Thread(target=join, daemon=True)
        t.start()
        while t.is_alive():
            t.join(0.1)
            why = self._dead_worker()
            if why is not None and t.is_alive():
                raise WorkerFailedError(why)             # the helper thread stays behind, blocked
        if "error" in result:
            raise WorkerFailedError(f"joining the RPC group failed: {result['error']}")

    def _recv_hello(self, rank: int, pipe: Pipe):
        while True:
            try:
                return pipe.recv(timeout=0.1)
            except RuntimeError:
                why = self._dead_worker()
                if why is not None:
                    self._abandon_rpc()
                    raise WorkerFailedError(why) from None

    def _abandon_rpc(self) -> None:
        for i in range(self.world_size):
            try:
                trpc.rpc_async(f"worker{i}", _request_stop, timeout=2.0)
            except Exception:                            # noqa: BLE001
                pass
        try:
            trpc.shutdown(graceful=False)
        except Exception:                                # noqa: BLE001
            pass

    def _submit_loop(self) -> None:
        while True:
            with self.work:
                while self.running and not self.submit_queue:
                    self.work.wait(0.1)
                if not self.running:
                    return
                task_entry, info = self.batch_manager.make_batch(self.submit_queue)
                self.batch_info[task_entry.uids] = (info, len(task_entry.uids), time.time())
            try:
                for pipe in self.submit_pipes:           # the same batch goes to every tensor-parallel rank
                    pipe.send(task_entry)
            except Exception as exc:                     # the peer is gone: RPC raises instead of delivering
                self._fail(f"sending a batch to a worker failed: {type(exc).__name__}: {exc}")
                return

    def _fail(self, why: str) -> None:
        with self.lock:
            if self.failed is None:
                self.failed = why

    def _check_workers(self) -> None:
        for rank, proc in enumerate(self.worker_procs):
            if proc.exitcode is not None and self.running:
                self._fail(f"worker process {rank} exited with code {proc.exitcode}")

    def _recv(self, pipe: Pipe):
        """Next item of a completion pipe, or None once the engine stops or has failed."""
        while self.running and self.failed is None:
            try:
                return pipe.recv(timeout=0.1)
            except RuntimeError:
                self._check_workers()
        return None

    def _completion_loop(self) -> None:
        while self.running and self.failed is None:
            copies = [self._recv(pipe) for pipe in self.completion_pipes]    # every rank's copy of one batch
            if any(c is None for c in copies):
                return
            first: TaskEntry = copies[0]
            failure = next((c.batch for c in copies if isinstance(c.batch, RemoteFailure)), None)
            with self.lock:
                info, _, _ = self.batch_info.pop(first.uids)
                if failure is not None:
                    for uid in first.uids:
                        self.completion_map[uid] = failure
                else:
                    for uid, output in self.batch_manager.split_batch(first, **info):
                        self.completion_map[uid] = output

    def submit(self, uid: Hashable, data: Any) -> None:
        if self.failed is not None:
            raise WorkerFailedError(self.failed)
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
                out = self.completion_map.pop(uid)
                if isinstance(out, RemoteFailure):
                    raise RuntimeError(f"request {uid!r} failed on worker {out.rank}: {out.message}")
                return True, out
            if self.failed is not None:
                raise WorkerFailedError(self.failed)
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
        if self.failed is None:
            self._check_workers()
        if self.failed is None:
            for i in range(self.world_size):
                trpc.rpc_sync(f"worker{i}", _request_stop)
            trpc.shutdown()
        else:
            # a peer is gone: ask the others to stop without waiting for answers, and do not
            # wait for the dead one in the RPC layer's own farewell round
            for i in range(self.world_size):
                try:
                    trpc.rpc_async(f"worker{i}", _request_stop, timeout=2.0)
                except Exception:
                    pass
            trpc.shutdown(graceful=False)
        self.submit_thread.join()
        self.completion_thread.join()
        for proc in self.worker_procs:
            proc.join(timeout=10)


def launch_engine(tp_world_size: Optional[int] = None, pp_world_size: int = 1, master_host: str = "127.0.0.1",
                  master_port: int = 29500, rpc_port: int = 29501, model_fn: Callable[..., nn.Module] = None,
                  n_nodes: int = 1, node_rank: int = 0, batch_manager: Optional[BatchManager] = None, pipe_size: int = 1,
                  queue_size: int = 0, rpc_disable_shm: bool = True, tp_init_size: Optional[int] = None,
                  pp_init_size: Optional[int] = None, **model_kwargs: Any) -> Optional[AsyncEngine]:
    """energonai/engine.py:157-168, same positional order.  `tp_init_size` / `pp_init_size` (the
    names of the reference's older server configurations) are accepted for the two sizes."""
    if tp_world_size is None:
        tp_world_size = 1 if tp_init_size is None else tp_init_size
    elif tp_init_size is not None and tp_init_size != tp_world_size:
        raise ValueError(f"tp_world_size={tp_world_size} and tp_init_size={tp_init_size} disagree")
    if pp_init_size is not None:
        pp_world_size = pp_init_size
    if model_fn is None:
        raise TypeError("launch_engine needs model_fn")
    world_size = tp_world_size * pp_world_size
    assert world_size % n_nodes == 0
    n_proc_per_node = world_size // n_nodes
    procs = launch_workers(tp_world_size, pp_world_size, master_host, master_port, rpc_port, model_fn,
                           n_proc_per_node=n_proc_per_node, node_rank=node_rank, pipe_size=pipe_size,
                           rpc_disable_shm=rpc_disable_shm, **model_kwargs)
    if node_rank == 0:
        return AsyncEngine(tp_world_size, pp_world_size, master_host, rpc_port, n_proc_per_node,
                           batch_manager=batch_manager, pipe_size=pipe_size, queue_size=queue_size,
                           rpc_disable_shm=rpc_disable_shm, worker_procs=procs)
    return None
