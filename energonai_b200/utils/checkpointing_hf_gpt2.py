"""Names and layouts of a Hugging Face GPT-2 checkpoint -> this package's PipelineModel.

Mirrors energonai/utils/checkpointing_hf_gpt2.py:29-91.  GPT-2 stores its projections as
Conv1D weights [in, out]; the four projection weights are transposed to [out, in], and the
fused c_attn weight and bias are cut into the unfused query_ / key_ / value_ entries (the
checkpoint's order is q, k, v).  The causal-mask buffers (`.attn.bias`) are dropped.
"""
import re
from collections import OrderedDict

import torch

__all__ = ["processing_HF_GPT"]

_LAYER = re.compile(r"h\.(\d+)?\.")
_SUBSTRINGS = (
    ("ln_2", "norm2"),
    ("c_attn", "query_key_value"),
    ("attn.c_proj", "attn.dense"),
    ("ln_1", "norm1"),
    ("c_fc", "dense_1"),
    ("mlp.c_proj", "mlp.dense_2"),
)
_TRANSPOSED = ("attn.query_key_value.weight", "mlp.dense_1.weight", "mlp.dense_2.weight", "attn.dense.weight")
_BLOCK_PREFIX = re.compile(r"blocks\.\d+?\.")


def _gpt2_name(key):
    """None for entries that are not parameters of the model."""
    if key == "wte.weight":
        return "embed.word_embeddings.weight"
    if key == "wpe.weight":
        return "embed.position_embeddings.weight"
    if "ln_f" in key:
        return key.replace("ln_f", "norm")
    if ".attn.bias" in key:
        return None
    key = _LAYER.sub(lambda m: f"blocks.{m.group(1)}.", key)
    for old, new in _SUBSTRINGS:
        key = key.replace(old, new)
    return key


def processing_HF_GPT(state_dict):
    """Returns {"model": renamed state dict, "epoch": 0}, the wrapper the reference returns;
    `load_checkpoint` unwraps it."""
    if "model" in state_dict:
        state_dict = state_dict.pop("model")
    out = OrderedDict()
    for key, value in state_dict.items():
        name = _gpt2_name(key)
        if name is None:
            continue
        if any(w in name for w in _TRANSPOSED):
            value = value.transpose(0, 1)
        fused = re.search(r"attn\.query_key_value\.(weight|bias)$", name)
        if fused:
            block = _BLOCK_PREFIX.search(name)
            prefix = block.group() if block else ""
            for part, piece in zip(("query_", "key_", "value_"), torch.chunk(value, 3, 0)):
                out[f"{prefix}attn.{part}.{fused.group(1)}"] = piece
        else:
            out[name] = value
    out["head.dense.weight"] = out["embed.word_embeddings.weight"].clone()
    return {"model": out, "epoch": 0}
