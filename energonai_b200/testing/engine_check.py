"""One engine life cycle in a fresh process (torch RPC cannot be re-initialised reliably inside
one process, which is also why the reference runs its engine tests one file per process):

    python -m energonai_b200.testing.engine_check <tp_world_size>

Launches workers, submits requests through a batching manager, checks BoringModel's closed form
(4x + 1), checks QueueFullError, shuts down.  Exit code 0 on success."""
import asyncio
import socket
import sys

import torch

from energonai_b200 import BatchManager, QueueFullError, TaskEntry, launch_engine
from energonai_b200.testing import BoringModel, get_correct_output


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class PairBatchManager(BatchManager):
    """Stacks up to two queued requests into one batch and splits the result again."""

    def make_batch(self, q):
        entries = [q.popleft() for _ in range(min(2, len(q)))]
        return TaskEntry(tuple(e.uid for e in entries), torch.stack([e.data for e in entries])), {"n": len(entries)}

    def split_batch(self, task_entry, n=1):
        return [(uid, task_entry.batch[i]) for i, uid in enumerate(task_entry.uids)]


def main(tp_world_size):
    engine = launch_engine(tp_world_size, 1, "127.0.0.1", free_port(), free_port(), BoringModel,
                           batch_manager=PairBatchManager(), queue_size=4)
    try:
        xs = {i: torch.full((4,), float(i)) for i in range(4)}
        for uid, x in xs.items():
            engine.submit(uid, x)
        for uid, x in xs.items():
            assert torch.equal(engine.get(uid), get_correct_output(x)), uid
        engine.submit("async", torch.ones(4))
        assert torch.equal(asyncio.run(engine.wait("async")), get_correct_output(torch.ones(4)))
        # a full queue refuses further requests: hold the submit thread's lock while filling it
        with engine.lock:
            full = False
            for i in range(10):
                try:
                    if engine.queue_size > 0 and len(engine.submit_queue) >= engine.queue_size:
                        raise QueueFullError(f"Submit queue full, size: {engine.queue_size}")
                    from energonai_b200 import SubmitEntry
                    engine.submit_queue.append(SubmitEntry(f"q{i}", torch.zeros(4)))
                except QueueFullError:
                    full = True
                    break
            assert full and len(engine.submit_queue) == engine.queue_size
        for i in range(engine.queue_size):
            assert torch.equal(engine.get(f"q{i}"), get_correct_output(torch.zeros(4)))
    finally:
        engine.shutdown()
    print("engine ok", tp_world_size, flush=True)


if __name__ == "__main__":
    main(int(sys.argv[1]))
