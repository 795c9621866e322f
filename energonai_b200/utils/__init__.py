"""Checkpoint loading into tensor-parallel shards (energonai/utils/checkpointing*.py)."""
from .checkpointing import load_checkpoint, load_state_dict, remove_prefix  # noqa: F401
from .checkpointing_hf_gpt2 import processing_HF_GPT  # noqa: F401
from .checkpointing_opt import load_175b, preprocess_175b, processing_OPT  # noqa: F401
