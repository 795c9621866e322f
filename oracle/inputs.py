"""Seeded synthetic weights and inputs (test infrastructure; see oracle/__init__.py).

All draws come from one CPU `torch.Generator`, in a fixed order, so the same seed gives the
same tensors on every machine running the same torch build.  Conventions of the benchmark
configurations: weights N(0, 0.02); biases 0 and LayerNorm gamma=1, beta=0 unless `rich` is
set (rich=True draws non-trivial biases / gamma / beta so that tests exercise them).
"""
import torch

BLOCK_SHAPES = (
    ("norm1.weight", "ln_w"), ("norm1.bias", "ln_b"),
    ("q.weight", "hh"), ("q.bias", "h"), ("k.weight", "hh"), ("k.bias", "h"),
    ("v.weight", "hh"), ("v.bias", "h"), ("dense.weight", "hh"), ("dense.bias", "h"),
    ("norm2.weight", "ln_w"), ("norm2.bias", "ln_b"),
    ("fc1.weight", "fh"), ("fc1.bias", "f"), ("fc2.weight", "hf"), ("fc2.bias", "h"),
)


def _draw(gen, kind, h, f, rich, std):
    if kind == "hh":
        return torch.randn(h, h, generator=gen) * std
    if kind == "fh":
        return torch.randn(f, h, generator=gen) * std
    if kind == "hf":
        return torch.randn(h, f, generator=gen) * std
    n = f if kind == "f" else h
    if kind == "ln_w":
        return 1.0 + 0.1 * torch.randn(n, generator=gen) if rich else torch.ones(n)
    return 0.1 * torch.randn(n, generator=gen) if rich else torch.zeros(n)


def block_params(gen, hidden, ffn, rich=False, std=0.02):
    """Logical parameters of one block (names documented in oracle/layers.py), fp32."""
    return {name: _draw(gen, kind, hidden, ffn, rich, std) for name, kind in BLOCK_SHAPES}


def model_params(seed, vocab, max_pos, hidden, ffn, depth, rich=False, std=0.02):
    """Logical parameters of a whole decoder-only model, fp32."""
    gen = torch.Generator().manual_seed(seed)
    p = {"embed.word.weight": torch.randn(vocab, hidden, generator=gen) * std,
         "embed.pos.weight": torch.randn(max_pos, hidden, generator=gen) * std}
    for i in range(depth):
        for k, v in block_params(gen, hidden, ffn, rich, std).items():
            p[f"blocks.{i}.{k}"] = v
    p["norm.weight"] = _draw(gen, "ln_w", hidden, ffn, rich, std)
    p["norm.bias"] = _draw(gen, "ln_b", hidden, ffn, rich, std)
    p["head.weight"] = torch.randn(vocab, hidden, generator=gen) * std
    return p


def left_padded_prompts(seed, batch, padded_len, lo, hi, vocab):
    """Prompt lengths uniform in [lo, hi], left-padded to padded_len; ids uniform in
    [2, vocab).  Returns (input_ids int64 [B,S], attention_mask fp32 [B,S], lens int64 [B]).
    Padding positions hold id 1 and mask 0."""
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (batch,), generator=gen)
    ids = torch.randint(2, vocab, (batch, padded_len), generator=gen)
    pos = torch.arange(padded_len)[None, :]
    valid = pos >= (padded_len - lens)[:, None]
    ids = torch.where(valid, ids, torch.ones_like(ids))
    return ids, valid.to(torch.float32), lens


def right_padded_lengths(seed, batch, lo, hi):
    """Sequence lengths uniform in [lo, hi] for the valid-tokens-first (right-padded)
    layout the padding kernels assume."""
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (batch,), generator=gen).to(torch.int32)
