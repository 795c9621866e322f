"""Layer modules and model factories with the interfaces of the reference's `energonai.model`."""
from .attention import MultiHeadAttention1D
from .mlp import MLP1D, gelu_impl
from .endecoder import Block1D
from .embedding import Embedding1D
from .downstream import LMHead1D
from .model_factory import (PipelineModel, create_pipeline_model, gpt2_small, gpt2_large, gpt2_8B, gpt3, hf_gpt2,
                            bert_small, bert_large, bert_8B, bert_175B, opt_125M, opt_6B, opt_13B, opt_30B, opt_66B,
                            opt_175B)

__all__ = ["MultiHeadAttention1D", "MLP1D", "Block1D", "Embedding1D", "LMHead1D", "PipelineModel", "gelu_impl",
           "create_pipeline_model", "gpt2_small", "gpt2_large", "gpt2_8B", "gpt3", "hf_gpt2", "bert_small",
           "bert_large", "bert_8B", "bert_175B", "opt_125M", "opt_6B", "opt_13B", "opt_30B", "opt_66B", "opt_175B"]
