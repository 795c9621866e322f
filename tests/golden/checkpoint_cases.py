"""Synthetic checkpoints with the key names and tensor layouts of the formats the reference
converts (Hugging Face OPT, metaseq OPT, one resharded 175B part, Hugging Face GPT-2), at toy
sizes.  Shared by make_checkpoint_golden.py (which runs the reference's converters on them) and
by the tests (which run this package's converters on the same dictionaries)."""
import torch

H, F, V, P, L = 8, 32, 24, 12, 2      # hidden, ffn, vocabulary, positions, layers


def _t(gen, *shape):
    return torch.randn(*shape, generator=gen)


def _opt_layer(gen, prefix, fused_rows=None):
    d = {}
    for n in ("self_attn_layer_norm", "final_layer_norm"):
        d[f"{prefix}{n}.weight"], d[f"{prefix}{n}.bias"] = _t(gen, H), _t(gen, H)
    if fused_rows is None:
        for n in ("q_proj", "k_proj", "v_proj"):
            d[f"{prefix}self_attn.{n}.weight"], d[f"{prefix}self_attn.{n}.bias"] = _t(gen, H, H), _t(gen, H)
    else:
        d[f"{prefix}self_attn.qkv_proj.weight"] = _t(gen, fused_rows, H)
        d[f"{prefix}self_attn.qkv_proj.bias"] = _t(gen, fused_rows)
    d[f"{prefix}self_attn.out_proj.weight"], d[f"{prefix}self_attn.out_proj.bias"] = _t(gen, H, H), _t(gen, H)
    d[f"{prefix}fc1.weight"], d[f"{prefix}fc1.bias"] = _t(gen, F, H), _t(gen, F)
    d[f"{prefix}fc2.weight"], d[f"{prefix}fc2.bias"] = _t(gen, H, F), _t(gen, H)
    return d


def opt_hf(root="decoder.", final_norm="final_layer_norm", wrapped=False, with_version=False):
    gen = torch.Generator().manual_seed(21)
    d = {f"{root}embed_tokens.weight": _t(gen, V, H), f"{root}embed_positions.weight": _t(gen, P, H)}
    if with_version:
        d[f"{root}version"] = torch.tensor([3.0])
    for i in range(L):
        d.update(_opt_layer(gen, f"{root}layers.{i}."))
    d[f"{root}{final_norm}.weight"], d[f"{root}{final_norm}.bias"] = _t(gen, H), _t(gen, H)
    return {"model": d} if wrapped else d


def opt_175b_part():
    gen = torch.Generator().manual_seed(22)
    d = {"decoder.embed_tokens.weight": _t(gen, V, H), "decoder.embed_positions.weight": _t(gen, P, H)}
    for i in range(L):
        d.update(_opt_layer(gen, f"decoder.layers.{i}.", fused_rows=3 * H // 2))
    d["decoder.layer_norm.weight"], d["decoder.layer_norm.bias"] = _t(gen, H), _t(gen, H)
    return d


def gpt2_hf(wrapped=False):
    gen = torch.Generator().manual_seed(23)
    d = {"wte.weight": _t(gen, V, H), "wpe.weight": _t(gen, P, H)}
    for i in range(L):
        p = f"h.{i}."
        for n in ("ln_1", "ln_2"):
            d[f"{p}{n}.weight"], d[f"{p}{n}.bias"] = _t(gen, H), _t(gen, H)
        d[f"{p}attn.bias"] = torch.ones(1, 1, P, P)
        d[f"{p}attn.c_attn.weight"], d[f"{p}attn.c_attn.bias"] = _t(gen, H, 3 * H), _t(gen, 3 * H)
        d[f"{p}attn.c_proj.weight"], d[f"{p}attn.c_proj.bias"] = _t(gen, H, H), _t(gen, H)
        d[f"{p}mlp.c_fc.weight"], d[f"{p}mlp.c_fc.bias"] = _t(gen, H, F), _t(gen, F)
        d[f"{p}mlp.c_proj.weight"], d[f"{p}mlp.c_proj.bias"] = _t(gen, F, H), _t(gen, H)
    d["ln_f.weight"], d["ln_f.bias"] = _t(gen, H), _t(gen, H)
    return {"model": d} if wrapped else d


CASES = {
    # name: (builder, converter name)
    "opt_hf": (lambda: opt_hf(), "processing_OPT"),
    "opt_metaseq_wrapped": (lambda: opt_hf(final_norm="layer_norm", wrapped=True, with_version=True), "processing_OPT"),
    "opt_175b_part": (opt_175b_part, "preprocess_175b"),
    "gpt2_hf": (lambda: gpt2_hf(), "processing_HF_GPT"),
    "gpt2_hf_wrapped": (lambda: gpt2_hf(wrapped=True), "processing_HF_GPT"),
}


def summarise(state):
    """key -> [shape, sum of |x| weighted by position] in insertion order (the weights make the
    figure sensitive to a transpose)."""
    if isinstance(state.get("model"), dict):
        state = state["model"]
    out = []
    for k, v in state.items():
        flat = v.double().contiguous().view(-1)
        w = torch.arange(1, flat.numel() + 1, dtype=torch.double)
        out.append([k, list(v.shape), round(float((flat * w).sum()), 6)])
    return out
