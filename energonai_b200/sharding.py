"""Cut full (tensor-parallel size 1) weights into the shards one rank of a 1-D tensor-parallel
group holds, using the reference's state_dict names.

Column-parallel weights (query_/key_/value_, dense_1) are split on dim 0, row-parallel weights
(attn.dense, dense_2) on dim 1, their biases stay whole; LayerNorm parameters are replicated.
A fused query_key_value weight of the whole model is taken as [key | value | query] blocks of
`hidden` rows each (the chunk order of energonai/model/attention.py:75 at size 1); the shard of
rank r is the r-th slice of each of the three blocks, concatenated in the same order, so that
every rank owns whole heads."""
import torch


def _rows(w, r, t):
    n = w.shape[0] // t
    return w[r * n:(r + 1) * n]


def _cols(w, r, t):
    n = w.shape[1] // t
    return w[:, r * n:(r + 1) * n]


def shard_block_state(full, rank, world):
    """full: state_dict of one Block1D at tensor-parallel size 1 -> the same keys for `rank`."""
    out = {}
    for k, v in full.items():
        leaf = k.rsplit(".", 1)[-1]
        if "query_key_value" in k:
            h = v.shape[0] // 3
            parts = [_rows(v[i * h:(i + 1) * h], rank, world) for i in range(3)]
            out[k] = torch.cat(parts, 0)
        elif any(s in k for s in ("query_.", "key_.", "value_.", "dense_1.")):
            out[k] = _rows(v, rank, world)
        elif ("attn.dense." in k or "dense_2." in k) and leaf == "weight":
            out[k] = _cols(v, rank, world)
        else:
            out[k] = v
    return {k: v.contiguous() for k, v in out.items()}


def shard_model_state(full, rank, world, vocab_parallel=False):
    """State dict of a whole PipelineModel: blocks cut as above, final norm and position
    embeddings replicated; word embedding and LM head replicated, or with vocab_parallel cut
    into `world` row slices of the vocabulary."""
    blocks, rest = {}, {}
    for k, v in full.items():
        (blocks if k.startswith("blocks.") else rest)[k] = v
    out = dict(rest)
    if vocab_parallel:
        for k in ("embed.word_embeddings.weight", "head.dense.weight", "head.dense.bias"):
            if k in out:
                out[k] = _rows(out[k], rank, world).contiguous()
    out.update(shard_block_state(blocks, rank, world))
    return out
