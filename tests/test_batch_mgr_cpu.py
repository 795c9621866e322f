"""BatchManagerForGeneration (examples/opt/batch.py:6-59): merged, left-padded batches and the
split of the outputs equal the reference's on random request queues (live where a checkout of
the reference is present; the closed-form cases below hold everywhere); length buckets and the
scan window are additions with tests of their own."""
import importlib.util
import os
import random
from collections import deque

import pytest
import torch

from energonai_b200 import BatchManagerForGeneration, SubmitEntry
from oracle import ref_loader


def _request(rng, n=None, max_tokens=None, sampling=None):
    n = rng.randint(1, 40) if n is None else n
    top_k, top_p, temp = sampling if sampling else rng.choice([(1, None, None), (50, 0.9, 0.7)])
    return {"input_ids": [rng.randint(2, 999) for _ in range(n)], "attention_mask": [1] * n, "top_k": top_k,
            "top_p": top_p, "temperature": temp, "max_tokens": rng.randint(1, 6) if max_tokens is None else max_tokens}


def _queue(seed, count):
    rng = random.Random(seed)
    return [SubmitEntry(uid, _request(rng)) for uid in range(count)]


def _same(a, b):
    if isinstance(a, torch.Tensor):
        return isinstance(b, torch.Tensor) and a.dtype == b.dtype and torch.equal(a, b)
    return a == b


def test_closed_form_left_padding_and_split():
    mgr = BatchManagerForGeneration(max_batch_size=4, pad_token_id=1)
    mk = lambda ids, mt, k=1: {"input_ids": ids, "attention_mask": [1] * len(ids), "top_k": k, "top_p": None,  # noqa: E731
                               "temperature": None, "max_tokens": mt}
    q = deque([SubmitEntry("a", mk([5, 6, 7], 4)), SubmitEntry("b", mk([8], 2)), SubmitEntry("c", mk([9, 9], 5)),
               SubmitEntry("d", mk([3], 1))])
    task, info = mgr.make_batch(q)
    # "c" asks for more new tokens than the first request: the batch stops there and "c", "d" stay queued
    assert task.uids == ("a", "b") and [e.uid for e in q] == ["c", "d"]
    assert task.batch["input_ids"].tolist() == [[5, 6, 7], [1, 1, 8]]
    assert task.batch["attention_mask"].tolist() == [[1, 1, 1], [0, 0, 1]]
    assert task.batch["input_ids"].dtype == torch.long
    assert task.batch["max_tokens"] == 3 + 4 and info == {"trunc_lens": [7, 5]}
    assert (task.batch["top_k"], task.batch["top_p"], task.batch["temperature"]) == (1, None, None)
    task.batch = torch.arange(14).view(2, 7)                       # the engine stores the outputs here
    out = mgr.split_batch(task, **info)
    assert out[0][0] == "a" and out[0][1].tolist() == list(range(7))
    assert out[1][0] == "b" and out[1][1].tolist() == list(range(7, 12))
    # different sampling settings are never merged
    q = deque([SubmitEntry(0, mk([1], 3, k=1)), SubmitEntry(1, mk([1], 3, k=50))])
    assert mgr.make_batch(q)[0].uids == (0,)


@pytest.mark.parametrize("seed", range(6))
def test_equals_the_reference_example_live(seed):
    root = ref_loader.reference_root()
    if root is None or ref_loader.load_reference_model_package() is None:
        pytest.skip("reference checkout not present")
    spec = importlib.util.spec_from_file_location("ref_opt_batch", os.path.join(root, "examples", "opt", "batch.py"))
    ref_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_mod)
    from energonai import SubmitEntry as RefEntry
    entries = _queue(seed, 24)
    mine, ref = BatchManagerForGeneration(5, pad_token_id=3), ref_mod.BatchManagerForGeneration(5, pad_token_id=3)
    qa, qb = deque(entries), deque(RefEntry(e.uid, e.data) for e in entries)
    while qa:
        (ta, ia), (tb, ib) = mine.make_batch(qa), ref.make_batch(qb)
        assert ta.uids == tb.uids and ia == ib and len(qa) == len(qb)
        assert set(ta.batch) == set(tb.batch) and all(_same(ta.batch[k], tb.batch[k]) for k in ta.batch)
        outputs = torch.arange(len(ta.uids) * ta.batch["max_tokens"]).view(len(ta.uids), -1)
        ta.batch = tb.batch = outputs
        sa, sb = mine.split_batch(ta, **ia), ref.split_batch(tb, **ib)
        assert [u for u, _ in sa] == [u for u, _ in sb] and all(torch.equal(x[1], y[1]) for x, y in zip(sa, sb))
    assert not qb


def test_length_buckets_and_scan_window():
    rng = random.Random(4)
    greedy = (1, None, None)
    lens = [300, 20, 270, 500, 257, 1000, 30, 512]
    q = deque(SubmitEntry(i, _request(rng, n, max_tokens=8, sampling=greedy)) for i, n in enumerate(lens))
    mgr = BatchManagerForGeneration(max_batch_size=8, pad_token_id=0, bucket_size=256, scan_window=8)
    batches = []
    while q:
        task, info = mgr.make_batch(q)
        batches.append(task.uids)
        width = task.batch["input_ids"].shape[1]
        assert width % 256 == 0 and task.batch["max_tokens"] == width + 8 and info["trunc_lens"] == [width + 8] * len(task.uids)
        for row, uid in enumerate(task.uids):                       # every prompt sits at the right edge of its row
            n = lens[uid]
            assert width - 256 < n <= width
            assert task.batch["attention_mask"][row].tolist() == [0] * (width - n) + [1] * n
            assert not task.batch["input_ids"][row, :width - n].any()
    # one batch per 256-wide bucket, formed in order of each bucket's first request; requests
    # that were skipped over kept their order
    assert batches == [(0, 2, 3, 4, 7), (1, 6), (5,)]
    # without a scan window the first request that does not fit ends the batch
    q = deque(SubmitEntry(i, _request(rng, n, max_tokens=8, sampling=greedy)) for i, n in enumerate(lens))
    mgr = BatchManagerForGeneration(max_batch_size=8, bucket_size=256)
    assert mgr.make_batch(q)[0].uids == (0,) and [e.uid for e in q] == list(range(1, 8))
    # a window of 1 reaches request 2 over request 1, not further
    q = deque(SubmitEntry(i, _request(rng, n, max_tokens=8, sampling=greedy)) for i, n in enumerate(lens))
    mgr = BatchManagerForGeneration(max_batch_size=8, bucket_size=256, scan_window=1)
    assert mgr.make_batch(q)[0].uids == (0, 2, 3, 4) and [e.uid for e in q] == [1, 5, 6, 7]
