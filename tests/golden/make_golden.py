"""Generate the golden fixtures in this directory from the reference's own Python code.

Run where a checkout of the reference is available (see oracle/ref_loader.py):

    python tests/golden/make_golden.py

It imports the reference's `energonai.model` unchanged (tensor-parallel size 1, CPU, fp32)
through the colossalai stand-in, feeds it seeded weights/inputs from oracle/inputs.py and
stores the outputs.  The fixtures keep only outputs plus checksums of the seeded inputs, so
the tests regenerate the inputs from the same seeds and verify the checksums first.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import inputs, layers, ref_loader  # noqa: E402

BLOCK_CASES = {
    # name: (fused_qkv, apply_post_layernorm, is_decoder, activation, pad_side)
    "preln_decoder_fused": (True, False, True, "gelu_tanh", "left"),
    "preln_decoder_unfused": (False, False, True, "relu", "left"),
    "postln_encoder_fused": (True, True, False, "gelu", "right"),
}
# head dimension 64 (= hidden / heads), the smallest the fused attention kernels implement
BLOCK_DIMS = dict(hidden=256, heads=4, ffn=1024, B=3, S=12, steps=2)
TINY = dict(vocab=512, max_pos=64, hidden=128, heads=2, ffn=512, depth=2, B=4, S=16, new=8)
CFG1 = dict(vocab=50272, max_pos=2050, hidden=768, heads=12, ffn=3072, depth=12, B=8, S=128, new=32)


def checksum(params):
    return float(sum(v.double().abs().sum() for v in params.values()))


def block_case_inputs(name):
    d = BLOCK_DIMS
    seed = sorted(BLOCK_CASES).index(name) + 100
    gen = torch.Generator().manual_seed(seed)
    bp = inputs.block_params(gen, d["hidden"], d["ffn"], rich=True, std=0.08)
    x = torch.randn(d["B"], d["S"] + d["steps"], d["hidden"], generator=gen)
    lens = torch.tensor([d["S"], d["S"] - 5, 3])
    pos = torch.arange(d["S"])[None, :]
    if BLOCK_CASES[name][4] == "left":
        valid = pos >= (d["S"] - lens)[:, None]
    else:
        valid = pos < lens[:, None]
    return bp, x, valid.float()


def run_block_reference(model_pkg, name):
    from energonai.model.endecoder import Block1D
    fused, post_ln, is_dec, act, _ = BLOCK_CASES[name]
    d = BLOCK_DIMS
    bp, x, mask = block_case_inputs(name)
    blk = Block1D(hidden_size=d["hidden"], num_heads=d["heads"], mlp_ratio=d["ffn"] / d["hidden"],
                  activation=layers.ACTIVATIONS[act], dtype=torch.float32, apply_post_layernorm=post_ln,
                  max_seq_len=32, fused_qkv=fused, is_decoder=is_dec)
    missing = blk.load_state_dict(layers.block_to_reference_state(bp, fused), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    outs = []
    with torch.inference_mode():
        for step in range(d["steps"] + 1):
            S = d["S"] + step
            m = torch.cat([mask, torch.ones(d["B"], step)], 1)
            m4 = (1.0 - m.view(d["B"], 1, 1, S)) * -10000.0
            outs.append(blk(x[:, :S].clone(), m4, first_cache=(step == 0)).numpy().copy())
    return {"checksum": checksum(bp) + float(x.double().abs().sum()),
            **{f"out{i}": o for i, o in enumerate(outs)}}


def run_model_reference(model_pkg, cfg, seed):
    from energonai.model.model_factory import create_pipeline_model
    p = inputs.model_params(seed, cfg["vocab"], cfg["max_pos"], cfg["hidden"], cfg["ffn"], cfg["depth"])
    ids, mask, lens = inputs.left_padded_prompts(seed, cfg["B"], cfg["S"], max(2, cfg["S"] // 8), cfg["S"], cfg["vocab"])
    model = create_pipeline_model(depth=cfg["depth"], vocab_size=cfg["vocab"], hidden_size=cfg["hidden"],
                                  max_seq_len=cfg["max_pos"], num_heads=cfg["heads"],
                                  mlp_ratio=cfg["ffn"] / cfg["hidden"], activation=torch.nn.functional.relu,
                                  is_decoder=True, fused_qkv=False, dtype=torch.float32)
    res = model.load_state_dict(layers.model_to_reference_state(p, cfg["depth"], False), strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    torch.manual_seed(0)
    with torch.inference_mode():
        out = model(input_ids=ids.clone(), attention_mask=mask.clone(), max_tokens=cfg["S"] + cfg["new"], top_k=1)
    # the oracle restatement supplies per-step logits (the reference does not expose them)
    rec = {}
    with torch.inference_mode():
        out2 = layers.OracleModel(p, cfg["depth"], cfg["heads"], "relu").generate(ids, mask, cfg["S"] + cfg["new"], rec)
    assert torch.equal(out, out2), "oracle restatement disagrees with the reference on greedy tokens"
    logits = torch.stack(rec["logits"], 0)                       # [new, B, vocab]
    top2 = logits.topk(2, -1).values
    return {"checksum": checksum(p), "input_ids": ids.numpy(), "attention_mask": mask.numpy(),
            "tokens": out[:, cfg["S"]:].numpy(), "top2_margin": (top2[..., 0] - top2[..., 1]).numpy(),
            "last_hidden": torch.stack(rec["hidden"], 0).numpy().astype(np.float32)}


def main():
    pkg = ref_loader.load_reference_model_package()
    if pkg is None:
        raise SystemExit("reference checkout not found; set ENERGONAI_REFERENCE")
    blocks = {}
    for name in BLOCK_CASES:
        for k, v in run_block_reference(pkg, name).items():
            blocks[f"{name}.{k}"] = v
    np.savez_compressed(os.path.join(HERE, "block_small.npz"), **blocks)
    np.savez_compressed(os.path.join(HERE, "opt_tiny_generate.npz"), **run_model_reference(pkg, TINY, seed=7))
    r = run_model_reference(pkg, CFG1, seed=0)
    r.pop("last_hidden")
    np.savez_compressed(os.path.join(HERE, "cfg1_opt125m_generate.npz"), **r)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
