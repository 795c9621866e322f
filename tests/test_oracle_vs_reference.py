"""Live check of the oracle restatement against the reference's own Python, run only where
a checkout of the reference is present (skipped elsewhere; the committed fixtures under
tests/golden/ carry the same comparison to machines without the checkout)."""
import pytest
import torch

from oracle import inputs, layers, ref_loader

pkg = ref_loader.load_reference_model_package() if ref_loader.reference_root() else None
pytestmark = pytest.mark.skipif(pkg is None, reason="reference checkout not present")


@pytest.mark.parametrize("fused,post_ln,is_dec,act", [(True, False, True, "relu"), (False, False, True, "gelu_tanh"),
                                                       (True, True, False, "gelu")])
def test_block_live(fused, post_ln, is_dec, act):
    from energonai.model.endecoder import Block1D
    h, H, f, B, S = 96, 6, 384, 2, 10
    gen = torch.Generator().manual_seed(11)
    bp = inputs.block_params(gen, h, f, rich=True, std=0.08)
    x = torch.randn(B, S + 3, h, generator=gen)
    mask = torch.ones(B, S)
    mask[1, :4] = 0
    ref = Block1D(h, H, f / h, activation=layers.ACTIVATIONS[act], dtype=torch.float32, apply_post_layernorm=post_ln,
                  max_seq_len=64, fused_qkv=fused, is_decoder=is_dec)
    ref.load_state_dict(layers.block_to_reference_state(bp, fused))
    mine = layers.OracleBlock(bp, H, act, apply_post_layernorm=post_ln, is_decoder=is_dec, tp=2)
    with torch.inference_mode():
        for step in range(4):
            m = torch.cat([mask, torch.ones(B, step)], 1)
            m4 = (1.0 - m.view(B, 1, 1, S + step)) * -10000.0
            a = ref(x[:, :S + step].clone(), m4, first_cache=(step == 0))
            b = mine(x[:, :S + step], m4, first_cache=(step == 0))
            assert torch.allclose(a, b, atol=2e-5, rtol=1e-5)
