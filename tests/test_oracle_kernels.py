"""The NumPy restatements of the reference CUDA kernels against the known answers of the
reference's own kernel-test fixture and the identities its tests assert."""
import numpy as np
import pytest

from oracle import kernels_np as K

# tests/test_kernel/test_ft_transpose_pad.py:6-11 and test_transpose_pad_fusion_kernel.py:6-11
SEQ_LENS = [24, 127, 31, 65, 24, 127, 31, 65]
B, S, H, D = 8, 128, 12, 64


def test_build_padding_offsets_known_answer():
    valid, off = K.build_padding_offsets(SEQ_LENS, B, S)
    assert valid == 494
    assert off.dtype == np.int32 and off.shape == (494,)
    starts = np.concatenate([[0], np.cumsum(SEQ_LENS)[:-1]])
    assert [int(off[s]) for s in starts] == [0, 104, 105, 202, 265, 369, 370, 467]
    # serial definition of the kernel (one thread, transpose_pad_fusion_kernel.cu:118-131)
    exp, cum = [], 0
    for L in SEQ_LENS:
        exp += [cum] * L
        cum += S - L
    assert off.tolist() == exp


def test_ft_round_trip_fixture():
    rng = np.random.default_rng(0)
    valid, off = K.build_padding_offsets(SEQ_LENS, B, S)
    x = rng.random((B, S, H * D), dtype=np.float32)
    packed, mask_off = K.remove_padding(x, off, valid)
    assert np.array_equal(mask_off, off)
    k = 0
    for b, L in enumerate(SEQ_LENS):
        assert np.array_equal(packed[k:k + L], x[b, :L])
        k += L
    buf = np.zeros((B, H, S, D), np.float32)
    K.transpose_rebuild_padding(packed, buf, B, S, H, D, valid, off)
    ref = x.reshape(B, S, H, D).transpose(0, 2, 1, 3).copy()
    for b, L in enumerate(SEQ_LENS):
        ref[b, :, L:, :] = 0
    assert np.array_equal(buf, ref)
    back = K.transpose_remove_padding(buf, valid, B, S, H, D, off)
    assert np.array_equal(back[0], packed)
    rebuilt = K.rebuild_padding(back[0], off, valid, B, S)
    for b, L in enumerate(SEQ_LENS):
        assert np.array_equal(rebuilt[b, :L], x[b, :L])
        assert not rebuilt[b, L:].any()


def test_turbo_identity():
    # tests/test_kernel/test_transpose_pad_fusion_kernel.py:63-79
    rng = np.random.default_rng(1)
    x = np.zeros((B, S, H * D), np.float32)
    for b, L in enumerate(SEQ_LENS):
        x[b, :L] = rng.standard_normal((L, H * D))
    packed = np.concatenate([x[b, :L] for b, L in enumerate(SEQ_LENS)], 0)[None]
    ref = x.reshape(B, S, H, D).transpose(0, 2, 1, 3)
    padded = K.transpose_pad(packed.reshape(1, -1, H, D), B, S, SEQ_LENS, H, D)
    assert np.array_equal(padded, ref)
    depad = K.transpose_depad(ref, B, sum(SEQ_LENS), S, SEQ_LENS, H, D)
    assert np.array_equal(depad.reshape(1, -1, H * D), packed)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_softmax_properties(dtype):
    rng = np.random.default_rng(2)
    b, h, s = 3, 2, 9
    x = rng.standard_normal((b, h, s, s)).astype(dtype)
    lens = np.array([9, 4, 0], np.int32)
    y = K.scale_mask_softmax(x, lens, b, s, h)
    for bi in range(b):
        L = lens[bi]
        assert np.array_equal(y[bi, :, L:], x[bi, :, L:])            # untouched rows
        for i in range(L):
            row = y[bi, :, i].astype(np.float64)
            assert np.all(row[:, i + 1:] == 0)
            assert np.allclose(row.sum(-1), 1, atol=4e-3 if dtype == np.float16 else 1e-6)
            e = np.exp(x[bi, :, i, :i + 1].astype(np.float64))
            assert np.allclose(row[:, :i + 1], e / e.sum(-1, keepdims=True), atol=1e-3 if dtype == np.float16 else 1e-6)


def test_layer_norm_matches_torch():
    import torch
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 7, 48)).astype(np.float32)
    g, bta = rng.standard_normal(48).astype(np.float32), rng.standard_normal(48).astype(np.float32)
    y, mu, iv = K.layer_norm_fwd(x, g, bta, 1e-5)
    ref = torch.nn.functional.layer_norm(torch.from_numpy(x), (48,), torch.from_numpy(g), torch.from_numpy(bta), 1e-5)
    assert np.allclose(y, ref.numpy(), atol=1e-5)
    assert np.allclose(mu, x.reshape(-1, 48).mean(1), atol=1e-6)
    assert np.allclose(iv, 1 / np.sqrt(x.reshape(-1, 48).var(1) + 1e-5), rtol=1e-5)


def test_linear():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 3, 16)).astype(np.float16)
    w = rng.standard_normal((8, 16)).astype(np.float16)
    assert np.allclose(K.linear(x, w).astype(np.float32), x.astype(np.float32) @ w.astype(np.float32).T, atol=2e-2)


def test_fold_layernorm_identity():
    """Host-side preparation of eb_gemm_ln: LayerNorm(x) W^T + b equals
    rstd * (x W'^T - mean * colsum) + bias32 with the folded operands (checked in fp64 so that only
    the algebra is tested, not rounding)."""
    import torch
    from energonai_b200.gemm import fold_layernorm
    g = torch.Generator().manual_seed(12)
    M, N, K, eps = 5, 24, 64, 1e-5
    x = torch.randn(M, K, generator=g, dtype=torch.float64) * 3 + 1.5
    w = torch.randn(N, K, generator=g, dtype=torch.float64)
    b = torch.randn(N, generator=g, dtype=torch.float64)
    gamma = 1 + 0.3 * torch.randn(K, generator=g, dtype=torch.float64)
    beta = 0.3 * torch.randn(K, generator=g, dtype=torch.float64)
    w_f, colsum, bias32 = fold_layernorm(w, b, gamma, beta)
    assert w_f.dtype == w.dtype and colsum.dtype == torch.float32 and bias32.dtype == torch.float32
    mean = x.mean(1, keepdim=True)
    rstd = (x.var(1, unbiased=False, keepdim=True) + eps).rsqrt()
    got = rstd * (x @ w_f.t() - mean * colsum.double()) + bias32.double()
    want = torch.nn.functional.layer_norm(x, (K,), gamma, beta, eps) @ w.t() + b
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-5), (got - want).abs().max()
    # without a projection bias
    _, _, bias_only = fold_layernorm(w, None, gamma, beta)
    assert torch.allclose(bias_only.double(), w @ beta, atol=1e-5)
