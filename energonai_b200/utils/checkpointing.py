"""Load a checkpoint of the whole model into the tensor-parallel shards of this process.

Mirrors energonai/utils/checkpointing.py: `load_state_dict` (:22-44, a file or a directory of
files merged into one dict), `remove_prefix` (:47-53), `load_checkpoint` (:56-98, same
arguments: file, model, strict, preprocess_fn, and `prefix` among the keyword arguments).

The reference reads the files on rank 0 and lets the parallel layers scatter their shards and
broadcast the rest.  Here every rank maps the files (torch.load with mmap, so the pages are
shared through the page cache and nothing is read that is not used), cuts out its own rows and
columns (`energonai_b200.sharding`) and copies only those to its GPU: no collective, and the
load time does not grow with the number of ranks.
"""
import os
import re
from collections import OrderedDict
from concurrent.futures import ThreadPoolExecutor
from time import time

import torch

from ..sharding import shard_model_state
from ..tp import get_tp

__all__ = ["load_checkpoint", "load_state_dict", "remove_prefix"]


def _load_file(path):
    """One checkpoint file as CPU tensors, memory-mapped where the file format allows."""
    try:
        return torch.load(path, map_location="cpu", mmap=True, weights_only=True)
    except (RuntimeError, ValueError):
        # files written with the legacy (non-zip) serialisation cannot be mapped
        return torch.load(path, map_location="cpu", weights_only=True)


def load_state_dict(path):
    """A file, or a directory whose files are merged in name order.  LOAD_N_PROC (the
    reference's environment variable) sets how many files are opened at once."""
    if os.path.isfile(path):
        return _load_file(path)
    if not os.path.isdir(path):
        raise FileNotFoundError(f"checkpoint {path} is neither a file nor a directory")
    files = sorted(os.path.join(path, f) for f in os.listdir(path) if os.path.isfile(os.path.join(path, f)))
    workers = max(1, min(int(os.environ.get("LOAD_N_PROC", "1")), len(files)))
    merged = {}
    if workers > 1:
        with ThreadPoolExecutor(workers) as pool:
            parts = list(pool.map(_load_file, files))
    else:
        parts = (_load_file(f) for f in files)
    for part in parts:
        merged.update(part)
    return merged


def remove_prefix(state_dict, prefix):
    """Drops every occurrence of `prefix` (a trailing dot is added if missing) from the keys."""
    if not prefix.endswith("."):
        prefix += "."
    return OrderedDict((k.replace(prefix, ""), v) for k, v in state_dict.items())


_NORM_LEAF = re.compile(r"(^|\.)(norm\d?)\.(weight|bias)$")


def _reconcile_norm_names(state, wanted):
    """LayerNorm1D keeps its affine parameters one level down (`norm1.module.weight`); some of
    the reference's converters emit `norm1.weight`.  Entries whose only difference to a wanted
    name is that level are renamed."""
    wanted = set(wanted)
    out = OrderedDict()
    for k, v in state.items():
        if k not in wanted:
            alt = _NORM_LEAF.sub(lambda m: f"{m.group(1)}{m.group(2)}.module.{m.group(3)}", k)
            if alt in wanted:
                k = alt
        out[k] = v
    return out


def _is_vocab_parallel(model_state, full_state, world):
    key = "embed.word_embeddings.weight"
    if world == 1 or key not in model_state or key not in full_state:
        key = "head.dense.weight"
        if world == 1 or key not in model_state or key not in full_state:
            return False
    return model_state[key].shape[0] * world == full_state[key].shape[0]


def load_checkpoint(file, model, strict=True, preprocess_fn=None, **kwargs):
    """Loads `file` (whole-model weights) into `model`, which holds the shards of this rank of
    the installed tensor-parallel context.  Returns -1 like the reference (no epoch is kept)."""
    start = time()
    state = load_state_dict(file)
    if preprocess_fn is not None:
        state = preprocess_fn(state)
    if isinstance(state.get("model"), dict):      # wrapper of processing_HF_GPT
        state = state["model"]
    if kwargs.get("prefix"):
        state = remove_prefix(state, kwargs["prefix"])
    own = model.state_dict()
    state = _reconcile_norm_names(state, own.keys())
    tp = get_tp()
    if tp.world_size > 1:
        state = shard_model_state(state, tp.rank, tp.world_size,
                                  vocab_parallel=_is_vocab_parallel(own, state, tp.world_size))
    result = model.load_state_dict(state, strict=strict)
    if os.environ.get("EB_VERBOSE"):
        print(f"rank {tp.rank}: checkpoint {file} loaded in {time() - start:.3f} s")
    del result
    return -1
