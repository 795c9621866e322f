"""The torch restatement of the reference layer forward against fixtures produced by the
reference's own Python code (tests/golden/make_golden.py), at simulated tensor-parallel
degrees 1, 2 and 4."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from oracle import layers

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)


@pytest.mark.parametrize("tp", [1, 2, 4])
@pytest.mark.parametrize("name", sorted(mg.BLOCK_CASES))
def test_block_against_reference_fixture(name, tp):
    gold = np.load(os.path.join(HERE, "golden", "block_small.npz"))
    fused, post_ln, is_dec, act, _ = mg.BLOCK_CASES[name]
    d = mg.BLOCK_DIMS
    bp, x, mask = mg.block_case_inputs(name)
    assert abs(mg.checksum(bp) + float(x.double().abs().sum()) - float(gold[f"{name}.checksum"])) < 1e-6
    blk = layers.OracleBlock(bp, d["heads"], act, apply_post_layernorm=post_ln, is_decoder=is_dec, tp=tp)
    for step in range(d["steps"] + 1):
        S = d["S"] + step
        m = torch.cat([mask, torch.ones(d["B"], step)], 1)
        m4 = (1.0 - m.view(d["B"], 1, 1, S)) * -10000.0
        out = blk(x[:, :S], m4, first_cache=(step == 0))
        ref = torch.from_numpy(gold[f"{name}.out{step}"])
        assert out.shape == ref.shape
        assert torch.allclose(out, ref, atol=2e-5, rtol=1e-5), (name, tp, step, (out - ref).abs().max())


@pytest.mark.parametrize("tp", [1, 2])
def test_tiny_generation_against_reference_fixture(tp):
    from oracle import inputs
    gold = np.load(os.path.join(HERE, "golden", "opt_tiny_generate.npz"))
    c = mg.TINY
    p = inputs.model_params(7, c["vocab"], c["max_pos"], c["hidden"], c["ffn"], c["depth"])
    assert abs(mg.checksum(p) - float(gold["checksum"])) < 1e-6
    ids, mask = torch.from_numpy(gold["input_ids"]), torch.from_numpy(gold["attention_mask"])
    rec = {}
    out = layers.OracleModel(p, c["depth"], c["heads"], "relu", tp=tp).generate(ids, mask, c["S"] + c["new"], rec)
    assert np.array_equal(out[:, c["S"]:].numpy(), gold["tokens"])
    assert np.allclose(torch.stack(rec["hidden"], 0).numpy(), gold["last_hidden"], atol=1e-4)


def test_cfg1_generation_against_reference_fixture():
    """BASELINE configuration 1: OPT-125M, seed 0, batch 8, prompts left-padded to 128,
    32 greedy steps."""
    from oracle import inputs
    gold = np.load(os.path.join(HERE, "golden", "cfg1_opt125m_generate.npz"))
    c = mg.CFG1
    p = inputs.model_params(0, c["vocab"], c["max_pos"], c["hidden"], c["ffn"], c["depth"])
    assert abs(mg.checksum(p) - float(gold["checksum"])) < 1e-3
    ids, mask = torch.from_numpy(gold["input_ids"]), torch.from_numpy(gold["attention_mask"])
    with torch.inference_mode():
        out = layers.OracleModel(p, c["depth"], c["heads"], "relu").generate(ids, mask, c["S"] + c["new"])
    assert np.array_equal(out[:, c["S"]:].numpy(), gold["tokens"])
