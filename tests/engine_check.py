"""One engine life cycle in a fresh process (torch RPC cannot be re-initialised reliably inside
one process, which is also why the reference runs its engine tests one file per process):

    python tests/engine_check.py <tp_world_size> [generation|failure|unhealthy|startup]

Launches workers, submits requests through a batching manager, checks BoringModel's closed form
(4x + 1), checks QueueFullError, shuts down.  With `generation`, the engine runs
BatchManagerForGeneration (length buckets, scan window) in front of a model whose answer to a
request does not depend on its batch: every request gets its own prompt and its own number of
new tokens back, however the requests were grouped.  With `failure`, a request the model rejects
is answered with a RuntimeError while the worker keeps serving, and a worker process that dies
turns pending and later requests into WorkerFailedError instead of a hang; shutdown still
returns.  Exit code 0 on success."""
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


def main_generation(tp_world_size):
    import random
    from energonai_b200 import BatchManagerForGeneration
    from energonai_b200.testing.models import EchoGenerator, expected_new_tokens
    rng = random.Random(3)
    reqs = {}
    for uid in range(12):
        n = rng.randint(1, 40)
        reqs[uid] = dict(input_ids=[rng.randint(2, 999) for _ in range(n)], attention_mask=[1] * n, top_k=1, top_p=None,
                         temperature=None, max_tokens=rng.randint(1, 9))
    mgr = BatchManagerForGeneration(max_batch_size=4, pad_token_id=0, bucket_size=16, scan_window=4)
    engine = launch_engine(tp_world_size, 1, "127.0.0.1", free_port(), free_port(), EchoGenerator, batch_manager=mgr)
    try:
        for uid, r in reqs.items():
            engine.submit(uid, r)
        for uid, r in reqs.items():
            out = engine.get(uid)
            n, new = len(r["input_ids"]), r["max_tokens"]
            width = out.numel() - new
            assert width % 16 == 0 and width >= n, (uid, out.shape)
            assert not out[:width - n].any() and out[width - n:width].tolist() == r["input_ids"], uid
            want = expected_new_tokens(torch.tensor(sum(r["input_ids"])), torch.arange(new))
            assert torch.equal(out[width:], want), (uid, out[width:], want)
    finally:
        engine.shutdown()
    print("engine generation ok", tp_world_size, flush=True)


def main_failure():
    import time
    from energonai_b200 import WorkerFailedError
    from energonai_b200.testing.models import FlakyModel
    engine = launch_engine(tp_init_size=1, master_host="127.0.0.1", master_port=free_port(), rpc_port=free_port(),
                           model_fn=FlakyModel)
    try:
        engine.submit("ok", torch.ones(4))
        assert torch.equal(engine.get("ok"), get_correct_output(torch.ones(4)))
        engine.submit("rejected", torch.full((4,), -1.0))
        try:
            engine.get("rejected")
            raise AssertionError("a rejected request must raise")
        except RuntimeError as exc:
            assert "request rejected by the model" in str(exc) and "'rejected'" in str(exc), exc
        engine.submit("after", torch.zeros(4))                       # the worker is still serving
        assert torch.equal(engine.get("after"), get_correct_output(torch.zeros(4)))
        engine.submit("crash", torch.full((4,), -2.0))
        t0 = time.time()
        try:
            engine.get("crash")
            raise AssertionError("a dead worker must raise")
        except WorkerFailedError as exc:
            assert "exited with code 7" in str(exc) or "failed" in str(exc), exc
        assert time.time() - t0 < 30
        try:
            engine.submit("later", torch.ones(4))
            raise AssertionError("submitting to a failed engine must raise")
        except WorkerFailedError:
            pass
    finally:
        engine.shutdown()
    print("engine failure ok", flush=True)


def main_unhealthy():
    """A worker whose health check reports a fault answers that batch, and every later one, with
    an error instead of results it cannot vouch for."""
    from energonai_b200.testing.models import FlakyModel
    engine = launch_engine(1, 1, "127.0.0.1", free_port(), free_port(), FlakyModel)
    try:
        engine.submit("ok", torch.ones(4))
        assert torch.equal(engine.get("ok"), get_correct_output(torch.ones(4)))
        for uid, x in (("faulted", torch.full((4,), -3.0)), ("later", torch.ones(4))):
            engine.submit(uid, x)
            try:
                engine.get(uid)
                raise AssertionError(f"{uid}: a faulted worker must not return results")
            except RuntimeError as exc:
                assert "ran out" in str(exc), exc
    finally:
        engine.shutdown()
    print("engine unhealthy ok", flush=True)


def main_startup():
    """A model_fn that raises makes launch_engine raise instead of waiting forever."""
    import time
    from energonai_b200 import WorkerFailedError
    from energonai_b200.testing.models import FlakyModel
    t0 = time.time()
    try:
        launch_engine(1, 1, "127.0.0.1", free_port(), free_port(), FlakyModel, fail_at_start=True)
        raise AssertionError("launch_engine must raise when a worker cannot start")
    except WorkerFailedError as exc:
        assert "failed on purpose" in str(exc) or "during start-up" in str(exc), exc
    assert time.time() - t0 < 60
    print("engine startup ok", flush=True)


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "failure":
        main_failure()
    elif len(sys.argv) > 2 and sys.argv[2] == "unhealthy":
        main_unhealthy()
    elif len(sys.argv) > 2 and sys.argv[2] == "startup":
        main_startup()
    elif len(sys.argv) > 2 and sys.argv[2] == "generation":
        main_generation(int(sys.argv[1]))
    else:
        main(int(sys.argv[1]))
