"""GPU parity of the tcgen05 GEMM (eb_gemm) against an fp32 reference of the same product.

Tolerance: operands are fp16/bf16 and accumulation is fp32, so the only error against the
fp32 product of the same rounded operands is the final rounding of the output (half an ulp
of the output type, relative 2^-11 for fp16 and 2^-8 for bf16) plus fp32 summation-order
noise; the test allows 2x that."""
import pytest
import torch

pytestmark = pytest.mark.gpu

REL = {torch.float16: 2 ** -10, torch.bfloat16: 2 ** -7, torch.float32: 1e-5}


def reference(a, w, bias=None, act=None, residual=None):
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == "relu":
        y = torch.relu(y)
    elif act == "gelu_tanh":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == "gelu":
        y = torch.nn.functional.gelu(y)
    if residual is not None:
        y = y + residual.float()
    return y


def check_close(out, ref, dtype):
    assert out.shape == ref.shape
    err = (out.float() - ref).abs()
    bound = REL[dtype] * ref.abs() + 2e-4 * ref.abs().max().clamp_min(1e-3)
    bad = err > bound
    assert not bad.any(), f"max err {err.max().item():.4g} at {int(bad.sum())} elements (ref max {ref.abs().max().item():.4g})"


def status_ok():
    from energonai_b200.gemm import device_status
    st = device_status()
    assert st[0] == 0, f"device status {st}"


SHAPES = [
    (256, 256, 64), (128 + 1, 8, 8), (300, 520, 200), (1024, 1024, 1024), (2048, 768, 3072), (640, 15360 // 8, 5120),
    (4096, 5120, 640), (1000, 2056, 264),
    # decode orientation (M <= 128): one weight pass split over all SMs
    (1, 256, 128), (16, 256, 64), (16, 5120, 5120), (16, 2560, 5120), (8, 1536, 12288), (64, 1152, 9216),
    (33, 520, 200), (100, 1024, 1024), (128, 384, 512), (16, 8, 8),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_plain(M, N, K, dtype):
    from energonai_b200.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dtype)
    out = gemm(a, w)
    torch.cuda.synchronize()
    status_ok()
    check_close(out, reference(a, w), dtype)
    out2 = gemm(a, w)                  # deterministic
    assert torch.equal(out, out2)


@pytest.mark.parametrize("M", [16, 512])
@pytest.mark.parametrize("act", [None, "relu", "gelu_tanh", "gelu"])
def test_gemm_epilogue(M, act):
    from energonai_b200.gemm import gemm
    N, K, dtype = 1024, 512, torch.float16
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dtype)
    bias = torch.randn(N, device="cuda", generator=g).to(dtype)
    res = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    out = gemm(a, w, bias=bias, act=act, residual=res)
    check_close(out, reference(a, w, bias, act, res), dtype)
    out32 = gemm(a, w, bias=bias, act=act, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    check_close(out32, reference(a, w, bias, act), torch.float32)
    status_ok()


@pytest.mark.parametrize("rows", [1, 48])
def test_gemm_writes_into_a_cache_view(rows):
    """Row m of the result lands at [m // rows, pos + m % rows, col0:col0+N] of a
    [batch, max_len, width] cache, leaving everything else untouched."""
    from energonai_b200.gemm import gemm
    B, max_len, width, N, K, pos, col0 = 5, 64, 96, 64, 128, 7, 16
    dtype = torch.float16
    a = torch.randn(B * rows, K, device="cuda").to(dtype)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dtype)
    cache = torch.full((B, max_len, width), 3.0, device="cuda", dtype=dtype)
    view = cache[:, pos:, col0:]
    gemm(a, w, out=view, out_rows_per_batch=rows, out_batch_stride=cache.stride(0), out_ld=cache.stride(1))
    ref = reference(a, w).view(B, rows, N)
    check_close(cache[:, pos:pos + rows, col0:col0 + N], ref, dtype)
    keep = torch.ones_like(cache, dtype=torch.bool)
    keep[:, pos:pos + rows, col0:col0 + N] = False
    assert (cache[keep] == 3.0).all()


def test_gemm_strided_operand_and_linear_api():
    from energonai_b200.gemm import gemm
    from energonai_b200.kernel import linear, find_algo
    big = torch.randn(300, 1024, device="cuda").half()
    a = big[:, 256:768]                            # row stride 1024, K = 512
    w = (torch.randn(264, 512, device="cuda") * 0.05).half()
    check_close(gemm(a, w), reference(a, w), torch.float16)
    x = torch.randn(4, 16, 512, device="cuda").half()
    y = linear(x, w, find_algo())
    assert y.shape == (4, 16, 264)
    check_close(y.view(-1, 264), reference(x.view(-1, 512), w), torch.float16)


def test_linear_reference_fixture_tolerance():
    """tests/test_kernel/test_linear_func.py:7-29: [16,64,12288] x [49152,12288] fp16 against
    F.linear with the reference's own pass criteria."""
    from energonai_b200.kernel import linear
    inputs = torch.randn(16, 64, 12288, device="cuda").half()
    params = torch.randn(49152, 12288, device="cuda").half()
    target = torch.nn.functional.linear(inputs, params)
    out = linear(inputs, params)
    diff = (out - target).abs()
    assert diff.mean() <= 0.5 and diff.max() <= 15 and diff.max() / target.max() <= 0.05


def test_gemm_rejects_bad_arguments():
    from energonai_b200.gemm import gemm
    a = torch.randn(16, 12, device="cuda").half()
    w = torch.randn(8, 12, device="cuda").half()
    with pytest.raises(RuntimeError, match="multiples of 8"):
        gemm(a, w)
    with pytest.raises(RuntimeError):
        gemm(a.float(), w.float())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", [None, "relu"])
@pytest.mark.parametrize("M,N,K", [(16, 5120, 5120), (1, 256, 128), (16, 1920, 5120), (32, 1024, 768), (5, 520, 200),
                                   (16, 8, 8), (20, 2560, 1024)])
def test_gemm_ln_fold(M, N, K, act, dtype):
    """LayerNorm folded into the GEMM (eb_gemm_ln) against LayerNorm -> projection in fp32.

    Tolerance: besides the rounding of the output, the folded weights W * gamma are rounded to
    the operand type once more (relative 2^-11 / 2^-8 per weight, averaging out over K), while the
    normalised activations are NOT rounded as they are on the two-kernel path; the bound is
    twice the plain GEMM's."""
    from energonai_b200.gemm import gemm, fold_layernorm
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + 7 * K)
    x = (torch.randn(M, K, device="cuda", generator=g) * 2.0 + 0.7).to(dtype)
    x[:, 0] += 6.0                                             # an outlier column, as residual streams have
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dtype)
    b = torch.randn(N, device="cuda", generator=g).to(dtype)
    gamma = (1 + 0.2 * torch.randn(K, device="cuda", generator=g)).to(dtype)
    beta = (0.2 * torch.randn(K, device="cuda", generator=g)).to(dtype)
    r = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    eps = 1e-5
    w_f, colsum, bias32 = fold_layernorm(w, b, gamma, beta)
    out = gemm(x, w_f, act=act, residual=r, static_weight=True, ln_fold=(colsum, bias32, eps))
    torch.cuda.synchronize()
    status_ok()
    xn = torch.nn.functional.layer_norm(x.float(), (K,), gamma.float(), beta.float(), eps)
    ref = xn @ w.float().t() + b.float()
    if act == "relu":
        ref = torch.relu(ref)
    ref = ref + r.float()
    err = (out.float() - ref).abs()
    bound = 2 * REL[dtype] * ref.abs() + 4e-4 * ref.abs().max().clamp_min(1e-3) + 2 * REL[dtype] * (xn.abs() @ w.float().abs().t()) / K ** 0.5
    assert not (err > bound).any(), f"max err {err.max().item():.4g} (ref max {ref.abs().max().item():.4g})"
    # and against the two-kernel path, which rounds the normalised activations
    two = gemm(layer_norm_forward(x, gamma, beta, eps), w, bias=b, act=act, residual=r)
    tol = {torch.float16: 4e-3, torch.bfloat16: 3e-2}[dtype]
    row_err = (out.float() - two.float()).abs().amax(-1)
    assert (row_err <= tol * two.float().abs().amax(-1).clamp_min(1e-3)).all(), row_err.max().item()
    assert torch.equal(out, gemm(x, w_f, act=act, residual=r, static_weight=True, ln_fold=(colsum, bias32, eps)))


def test_gemm_ln_fold_rejects_wide_batches():
    from energonai_b200.gemm import gemm, fold_layernorm
    x = torch.zeros(33, 64, device="cuda", dtype=torch.float16)
    w = torch.zeros(64, 64, device="cuda", dtype=torch.float16)
    ones = torch.ones(64, device="cuda", dtype=torch.float16)
    w_f, colsum, bias32 = fold_layernorm(w, None, ones, ones)
    with pytest.raises(RuntimeError):
        gemm(x, w_f, ln_fold=(colsum, bias32, 1e-5))
