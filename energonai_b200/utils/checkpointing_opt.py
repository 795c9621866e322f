"""Names of OPT checkpoints -> names of this package's PipelineModel.

Mirrors energonai/utils/checkpointing_opt.py: `processing_OPT` (:56-106) renames a Hugging Face
or metaseq OPT state dict of the whole model, `preprocess_175b` (:114-135) renames one
tensor-parallel part of the resharded 175B checkpoint, `load_175b` (:138-143) copies such a
part into the parameters of the calling rank.  The renaming is written as ordered rule tables;
the result for every key is the one the reference's functions give (pinned by
tests/golden/checkpoint_names.json, generated from the reference's own code).
"""
import os
import re
from collections import OrderedDict

import torch

from ..tp import get_tp

__all__ = ["processing_OPT", "preprocess_175b", "load_175b"]

# whole-key matches first, then "contains" rules that stop the renaming, then the substring
# rules applied one after the other to every remaining key
_OPT_EXACT = {
    "decoder.embed_tokens.weight": "embed.word_embeddings.weight",
    "decoder.embed_positions.weight": "embed.position_embeddings.weight",
}
_OPT_FINAL_NORM = ("decoder.layer_norm", "decoder.final_layer_norm")   # metaseq / Hugging Face spelling
_OPT_LAYER = re.compile(r"decoder.layers\.(\d+)?\.")
_OPT_SUBSTRINGS = (
    ("embed_tokens", "embed.word_embeddings"),
    ("embed_positions", "embed.position_embeddings"),
    ("self_attn.q_proj", "attn.query_"),
    ("self_attn.k_proj", "attn.key_"),
    ("self_attn.v_proj", "attn.value_"),
    ("self_attn.out_proj", "attn.dense"),
    ("self_attn_layer_norm", "norm1.module"),
    ("final_layer_norm", "norm2.module"),
    ("fc1", "mlp.dense_1"),
    ("fc2", "mlp.dense_2"),
)


def _opt_name(key):
    if key in _OPT_EXACT:
        return _OPT_EXACT[key]
    for spelled in _OPT_FINAL_NORM:
        if spelled in key:
            return key.replace(spelled, "norm.module")
    key = _OPT_LAYER.sub(lambda m: f"blocks.{m.group(1)}.", key)
    for old, new in _OPT_SUBSTRINGS:
        key = key.replace(old, new)
    return key


def processing_OPT(state_dict):
    """Whole-model OPT state dict (optionally wrapped as {"model": ...}) -> reference names.
    The LM head is a parameter of its own: without one in the checkpoint it starts as a copy of
    the word embedding.  The metaseq bookkeeping entry `decoder.version` is dropped."""
    if "model" in state_dict:
        state_dict = state_dict.pop("model")
    out = OrderedDict((_opt_name(k), v) for k, v in state_dict.items())
    if "head.dense.weight" not in out:
        out["head.dense.weight"] = out["embed.word_embeddings.weight"].clone()
    out.pop("decoder.version", None)
    return out


_175B_SUBSTRINGS = (
    ("decoder.embed_tokens.weight", "embed.word_embeddings.weight"),
    ("decoder.embed_positions.weight", "embed.position_embeddings.weight"),
    ("decoder.layer_norm", "norm"),
    ("decoder.layers", "blocks"),
    ("self_attn.qkv_proj", "attn.query_key_value"),
    ("self_attn.out_proj", "attn.dense"),
    ("self_attn_layer_norm", "norm1"),
    ("final_layer_norm", "norm2"),
    ("fc1", "mlp.dense_1"),
    ("fc2", "mlp.dense_2"),
)


def preprocess_175b(state_dict):
    """One `reshard-model_part-<rank>.pt` of the 175B checkpoint -> reference names (the fused
    qkv_proj of a part is already this rank's key | value | query rows)."""
    out = {}
    for key, value in state_dict.items():
        for old, new in _175B_SUBSTRINGS:
            key = key.replace(old, new)
        out[key] = value
    out["head.dense.weight"] = out["embed.word_embeddings.weight"].clone()
    return out


def load_175b(checkpoint_dir, model):
    """Every rank maps its own part file and copies it into its parameters: no rank-0 load, no
    broadcast.  LayerNorm parameters are matched with or without the `.module` level of the
    LayerNorm1D wrapper."""
    from .checkpointing import _load_file, _reconcile_norm_names
    rank = get_tp().rank
    part = os.path.join(checkpoint_dir, f"reshard-model_part-{rank}.pt")
    state = _reconcile_norm_names(preprocess_175b(_load_file(part)), [n for n, _ in model.named_parameters()])
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name not in state:
                raise KeyError(f"{part}: no tensor for parameter {name}")
            if tuple(state[name].shape) != tuple(p.shape):
                raise RuntimeError(f"{part}: {name} has shape {tuple(state[name].shape)}, the model's shard is "
                                   f"{tuple(p.shape)}")
            p.copy_(state[name])
