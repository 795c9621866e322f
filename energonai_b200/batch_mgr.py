"""BatchManager / SubmitEntry with the reference's interface (energonai/batch_mgr.py:6-18):
the default manager forwards one request per batch; subclasses merge and split requests."""
from dataclasses import dataclass
from typing import Any, Deque, Hashable, Iterable, Tuple

from .task import TaskEntry


@dataclass
class SubmitEntry:
    uid: Hashable
    data: Any


class BatchManager:
    def make_batch(self, q: Deque[SubmitEntry]) -> Tuple[TaskEntry, dict]:
        entry = q.popleft()
        return TaskEntry((entry.uid,), entry.data), {}

    def split_batch(self, task_entry: TaskEntry, **kwargs: Any) -> Iterable[Tuple[Hashable, Any]]:
        return [(task_entry.uids[0], task_entry.batch)]
