"""TaskEntry with the reference's fields (energonai/task.py:5-8)."""
from dataclasses import dataclass
from typing import Any, Hashable, Tuple


@dataclass
class TaskEntry:
    uids: Tuple[Hashable, ...]
    batch: Any


@dataclass
class RemoteFailure:
    """What a worker sends back in place of a batch's outputs when the model raised: the
    requests of that batch are answered with an exception instead of never being answered."""
    rank: int
    message: str
