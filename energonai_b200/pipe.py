"""Named one-way queues between RPC peers (the role of energonai/pipe.py:20-75).

A pipe lives in the destination process as a `queue.Queue`; the source delivers with one
blocking RPC that puts into it (back-pressure comes from the queue's own bound), and the
destination blocks on `get` instead of polling."""
import queue
import threading
from typing import Any, Dict

import torch.distributed.rpc as trpc

_queues: Dict[str, "queue.Queue[Any]"] = {}
_lock = threading.Lock()


def _local_queue(name: str, max_size: int = 0) -> "queue.Queue[Any]":
    with _lock:
        q = _queues.get(name)
        if q is None:
            q = _queues[name] = queue.Queue(max_size)
        return q


def _deliver(name: str, data: Any) -> None:
    _local_queue(name).put(data)


class Pipe:
    def __init__(self, name: str, src: str, dest: str, max_size: int = 0) -> None:
        self.name, self.src, self.dest = name, src, dest
        self.me = trpc.get_worker_info().name
        if self.me == dest:
            self.queue = _local_queue(name, max_size)

    def send(self, data: Any) -> None:
        assert self.me == self.src, f"pipe {self.name}: only {self.src} may send"
        trpc.rpc_sync(self.dest, _deliver, args=(self.name, data))

    def recv(self, timeout=None) -> Any:
        """Blocks until an item arrives; raises RuntimeError('pipe is empty') after `timeout`."""
        assert self.me == self.dest, f"pipe {self.name}: only {self.dest} may receive"
        try:
            return self.queue.get(timeout=timeout)
        except queue.Empty:
            raise RuntimeError("pipe is empty") from None

    def recv_nowait(self) -> Any:
        assert self.me == self.dest
        try:
            return self.queue.get_nowait()
        except queue.Empty:
            raise RuntimeError("pipe is empty") from None
