"""Layer parity at the shapes of the benchmark configurations (reduced in batch / length only
where the CPU oracle would otherwise need minutes): BERT-large block with right padding and the
padding kernels (configuration 2), a GPT-3-175B-shaped layer (configuration 4), an
OPT-66B-shaped layer in bf16 with bucketed left padding (configuration 5), and
scale_mask_softmax at configuration 2's score shape.

Tolerance: |out - ref| <= 2e-2 + 1e-2*|ref| against the reference-restating fp32 oracle; bf16
relative to the row maximum (see tests/test_layers_gpu.py)."""
import numpy as np
import pytest
import torch

from oracle import inputs, layers
from oracle import kernels_np as K

pytestmark = pytest.mark.gpu


def close(out, ref, row_relative=False, rel=1e-2):
    out, ref = out.float().cpu(), ref.float().cpu()
    scale = ref.abs().amax(-1, keepdim=True) if row_relative else ref.abs()
    err = (out - ref).abs()
    worst = (err / (2e-2 + rel * scale)).max().item()
    assert worst <= 1.0, (f"max err {err.max():.4g}, {worst:.2f}x the bound; row maxima "
                          f"{ref.abs().amax(-1).min():.3g}..{ref.abs().amax(-1).max():.3g}")


def build(bp, h, H, f, act, dtype, fused, post_ln=False, is_decoder=True):
    from energonai_b200.model import Block1D
    blk = Block1D(h, H, f / h, activation=layers.ACTIVATIONS[act], dtype=dtype, fused_qkv=fused,
                  apply_post_layernorm=post_ln, is_decoder=is_decoder, disable_past_cache=not is_decoder).cuda()
    blk.load_state_dict({k: v.to(dtype) for k, v in layers.block_to_reference_state(bp, fused).items()})
    return blk


def test_config2_bert_large_block_with_padding_kernels():
    from energonai_b200 import kernel as EK
    h, H, f, B, S = 1024, 16, 4096, 32, 512
    gen = torch.Generator().manual_seed(1)
    bp = inputs.block_params(gen, h, f)
    lens = inputs.right_padded_lengths(1, B, 32, S)
    x = torch.randn(B, S, h, generator=gen)
    valid = torch.arange(S)[None, :] < lens[:, None]
    x = x * valid[:, :, None]
    m4 = (1.0 - valid.float().view(B, 1, 1, S)) * -10000.0
    blk = build(bp, h, H, f, "gelu", torch.float16, True, post_ln=True, is_decoder=False)
    with torch.inference_mode():
        out = blk(x.half().cuda(), m4.half().cuda())
        ref = layers.OracleBlock(bp, H, "gelu", apply_post_layernorm=True, is_decoder=False)(x, m4, True)
    close(out, ref)
    # the packed (padding-removed) view of the block output, through the FT kernels
    lens_d = lens.cuda()
    valid_n = torch.zeros(1, dtype=torch.int32, device="cuda")
    tmp = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    moff = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    EK.ft_build_padding_offsets(lens_d, B, S, valid_n, tmp)
    V = int(valid_n.item())
    assert V == int(lens.sum())
    packed = EK.ft_remove_padding(out, tmp, moff, V, h)
    assert torch.equal(packed[0], out[valid.cuda()])
    rebuilt = EK.ft_rebuild_padding(packed, moff, V, h, B, S)
    assert torch.equal(rebuilt[valid.cuda()], out[valid.cuda()]) and not rebuilt[~valid.cuda()].any()
    heads = EK.ft_transpose_remove_padding(out.view(B, S, H, h // H).permute(0, 2, 1, 3).contiguous(), V, B, S, H, h // H, moff)
    assert torch.equal(heads, packed)


def test_config2_scale_mask_softmax_shape():
    from energonai_b200.kernel import scale_mask_softmax
    B, H, S = 8, 16, 512
    rng = np.random.default_rng(2)
    x = rng.standard_normal((B, H, S, S)).astype(np.float16)
    lens = rng.integers(32, S + 1, B).astype(np.int32)
    out = scale_mask_softmax(B, S, H, torch.from_numpy(x).cuda(), torch.from_numpy(lens).cuda()).cpu().numpy()
    ref = K.scale_mask_softmax(x, lens, B, S, H)
    assert np.abs(out.astype(np.float32) - ref.astype(np.float32)).max() <= 1e-3
    for b in range(B):
        assert np.array_equal(out[b, :, lens[b]:], x[b, :, lens[b]:])


@pytest.mark.parametrize("name,h,H,f,act,fused,dtype,B,S", [
    ("config4 GPT-3 layer", 12288, 96, 49152, "gelu_tanh", True, torch.float16, 1, 64),
    ("config5 OPT-66B layer", 9216, 72, 36864, "relu", False, torch.bfloat16, 4, 96),
])
def test_large_layer_shapes(name, h, H, f, act, fused, dtype, B, S):
    gen = torch.Generator().manual_seed(0)
    bp = inputs.block_params(gen, h, f)
    x = torch.randn(B, S + 2, h, generator=gen)
    lens = torch.tensor([S] + [max(8, S - 17 * i) for i in range(1, B)])
    mask = (torch.arange(S)[None, :] >= (S - lens)[:, None]).float()
    blk = build(bp, h, H, f, act, dtype, fused)
    ref = layers.OracleBlock(bp, H, act)
    # With hidden sizes of 9k-12k and N(0, 0.02) weights the block output has a standard deviation
    # of ~5 and row maxima of 20-30, where one fp16 ulp is already 1.6e-2 (bf16: 1.3e-1): the
    # absolute part of the tolerance cannot hold element-wise, so the relative part is taken
    # against the row maximum for both dtypes here.  bf16 keeps three mantissa bits fewer than
    # fp16; its relative part is 2e-2 of the row maximum (about 4 bf16 ulps at that magnitude;
    # measured worst case 1.3e-2).
    rr = True
    rel = 2e-2 if dtype == torch.bfloat16 else 1e-2
    with torch.inference_mode():
        for step in range(3):
            cur = S + step
            m = torch.cat([mask, torch.ones(B, step)], 1)
            m4 = (1.0 - m.view(B, 1, 1, cur)) * -10000.0
            out = blk(x[:, :cur].to(dtype).cuda(), m4.to(dtype).cuda(), first_cache=(step == 0))
            exp = ref(x[:, :cur], m4, step == 0)
            if step == 0:
                close(out.cpu()[m.bool()], exp[m.bool()], rr, rel)
            else:
                close(out[:, -1], exp[:, -1], rr, rel)
