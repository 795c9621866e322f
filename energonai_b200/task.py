"""TaskEntry with the reference's fields (energonai/task.py:5-8)."""
from dataclasses import dataclass
from typing import Any, Hashable, Tuple


@dataclass
class TaskEntry:
    uids: Tuple[Hashable, ...]
    batch: Any
