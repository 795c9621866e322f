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


class BatchManagerForGeneration(BatchManager):
    """Merges queued generation requests into one left-padded batch and cuts the outputs apart
    again (examples/opt/batch.py:6-59, same constructor arguments, same make_batch /
    split_batch results).

    A request is a dict with `input_ids`, `attention_mask` (lists), `top_k`, `top_p`,
    `temperature`, `max_tokens`.  Requests are merged while they share the sampling settings of
    the first one and ask for no more new tokens than it (the batch runs for the first
    request's `max_tokens`).  Padding goes on the left with attention_mask 0, so every prompt
    ends at the same column and the generation loop appends behind it.

    Two additions, both off by default (then the batches are exactly the reference's):

    * `bucket_size`: the padded length is rounded up to a multiple of it, and only requests
      whose own length falls into the first request's bucket are merged.  Prompt lengths then
      take few distinct values, so prompt-pass kernels, key/value cache capacities and captured
      generation-step graphs are reused across batches instead of being set up per length.
    * `scan_window`: how many queued requests beyond the next one may be skipped over while
      looking for mergeable ones (0 = stop at the first request that does not fit, like the
      reference).  Skipped requests keep their order.
    """

    def __init__(self, max_batch_size: int = 1, pad_token_id: int = 0, bucket_size: int = 0,
                 scan_window: int = 0) -> None:
        super().__init__()
        self.max_batch_size, self.pad_token_id = max_batch_size, pad_token_id
        self.bucket_size, self.scan_window = int(bucket_size), int(scan_window)

    def _bucket(self, n):
        b = self.bucket_size
        return n if b <= 0 else max(b, -(-n // b) * b)

    def _left_padding(self, batch_inputs):
        import torch
        lens = [len(d["input_ids"]) for d in batch_inputs]
        width = self._bucket(max(lens))
        ids = torch.full((len(lens), width), self.pad_token_id, dtype=torch.long)
        mask = torch.zeros((len(lens), width), dtype=torch.long)
        for row, (d, n) in enumerate(zip(batch_inputs, lens)):
            if n:
                ids[row, width - n:] = torch.as_tensor(d["input_ids"], dtype=torch.long)
                mask[row, width - n:] = torch.as_tensor(d["attention_mask"], dtype=torch.long)
        return {"input_ids": ids, "attention_mask": mask}, width

    @staticmethod
    def _make_batch_key(entry: SubmitEntry) -> tuple:
        d = entry.data
        return (d["top_k"], d["top_p"], d["temperature"])

    def _fits(self, head: SubmitEntry, other: SubmitEntry) -> bool:
        if self._make_batch_key(head) != self._make_batch_key(other):
            return False
        if other.data["max_tokens"] > head.data["max_tokens"]:
            return False
        if self.bucket_size > 0:
            return self._bucket(len(other.data["input_ids"])) == self._bucket(len(head.data["input_ids"]))
        return True

    def make_batch(self, q: Deque[SubmitEntry]) -> Tuple[TaskEntry, dict]:
        head = q.popleft()
        taken, skipped = [head], []
        while len(taken) < self.max_batch_size and q:
            if self._fits(head, q[0]):
                taken.append(q.popleft())
            elif len(skipped) < self.scan_window:
                skipped.append(q.popleft())
            else:
                break
        q.extendleft(reversed(skipped))
        inputs, width = self._left_padding([e.data for e in taken])
        for k in ("top_k", "top_p", "temperature"):
            inputs[k] = head.data[k]
        inputs["max_tokens"] = width + head.data["max_tokens"]
        trunc_lens = [width + e.data["max_tokens"] for e in taken]
        return TaskEntry(tuple(e.uid for e in taken), inputs), {"trunc_lens": trunc_lens}

    def split_batch(self, task_entry: TaskEntry, trunc_lens=()) -> Iterable[Tuple[Hashable, Any]]:
        return [(uid, out[:n]) for uid, out, n in zip(task_entry.uids, task_entry.batch, trunc_lens)]
