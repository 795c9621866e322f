"""GPU parity of the fused attention kernels against an fp32 restatement of
energonai/model/attention.py:105-118 evaluated on the same (rounded) inputs.

Tolerance: probabilities are rounded to the tensor dtype before the value product (as in the
reference, attention.py:116) and the output is rounded once; with |v| ~ 1 that is a few
ulps of the output type: 4e-3 for fp16, 3e-2 for bf16."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 4e-3, torch.bfloat16: 3e-2}


def reference(q, k, v, D, mask, causal):
    """q [B,Sq,H*D], k/v [B,Sk,H*D], mask [B,Sk] additive.  fp32 math throughout."""
    B, Sq, HD = q.shape
    Sk, H = k.shape[1], HD // D
    qf, kf, vf = (t.float().view(B, -1, H, D).permute(0, 2, 1, 3) for t in (q, k, v))
    s = (qf * D ** -0.5) @ kf.transpose(-1, -2)
    if causal:
        tril = torch.tril(torch.ones(Sq, Sk, dtype=torch.bool, device=q.device), diagonal=Sk - Sq)
        s = torch.where(tril, s, torch.tensor(-1e4, device=q.device))
    if mask is not None:
        s = s + mask.float().view(B, 1, 1, Sk)
    p = torch.softmax(s, -1)
    return (p @ vf).permute(0, 2, 1, 3).reshape(B, Sq, HD)


def make_mask(B, S, lens, side, dtype):
    pos = torch.arange(S, device="cuda")[None, :]
    lens = torch.tensor(lens, device="cuda")[:, None]
    valid = pos >= (S - lens) if side == "left" else pos < lens
    return ((1.0 - valid.float()) * -10000.0).to(dtype), valid


@pytest.mark.parametrize("impl", ["mma", "tc"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,S,D,causal,side", [
    (2, 3, 128, 64, True, "left"), (3, 2, 200, 128, True, "left"), (2, 2, 65, 64, True, None),
    (2, 4, 512, 128, True, "left"), (3, 2, 96, 64, False, "right"), (2, 2, 333, 128, False, "right"),
    (1, 1, 1, 64, True, None), (1, 2, 1024, 128, True, None),
])
def test_prefill(B, H, S, D, causal, side, dtype, impl):
    from energonai_b200.attention import attention_prefill
    g = torch.Generator(device="cuda").manual_seed(S + D)
    qkv = torch.randn(B, S, 3 * H * D, device="cuda", generator=g).to(dtype)      # fused k|v|q buffer: strided views
    k, v, q = qkv[:, :, :H * D], qkv[:, :, H * D:2 * H * D], qkv[:, :, 2 * H * D:]
    mask, valid = (None, None)
    if side:
        lens = [S] + [max(1, S // (i + 2)) for i in range(B - 1)]
        mask, valid = make_mask(B, S, lens, side, dtype)
    out = attention_prefill(q, k, v, D, mask=mask, causal=causal, impl=impl)
    ref = reference(q, k, v, D, mask, causal)
    err = (out.float() - ref).abs()
    if side == "left":          # rows of left-padding queries are unspecified (never consumed): compare valid rows
        err = err * valid[:, :, None]
    assert err.max().item() <= TOL[dtype], err.max().item()
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,Sq,Sk,D,causal", [(2, 3, 100, 356, 128, True), (1, 5, 260, 300, 64, True), (2, 2, 129, 40, 64, False),
                                                (16, 5, 512, 512, 128, True)])
def test_prefill_tc_rectangular(B, H, Sq, Sk, D, causal, dtype):
    """Tensor-core prompt kernel with q_len != kv_len (a prompt continued against cached keys),
    separate q / k / v / out tensors, a right-side key mask, and the two kernels against each other."""
    from energonai_b200.attention import attention_prefill
    from energonai_b200._lib import lib
    import ctypes
    g = torch.Generator(device="cuda").manual_seed(Sq * 7 + Sk)
    q = torch.randn(B, Sq, H * D, device="cuda", generator=g).to(dtype)
    k = torch.randn(B, Sk, H * D, device="cuda", generator=g).to(dtype)
    v = torch.randn(B, Sk, H * D, device="cuda", generator=g).to(dtype)
    lens = [Sk] + [max(Sk - Sq + 1, Sk - 3 * (i + 1)) for i in range(B - 1)]
    mask, _ = make_mask(B, Sk, lens, "right", dtype)
    out = attention_prefill(q, k, v, D, mask=mask, causal=causal, impl="tc")
    ref = reference(q, k, v, D, mask, causal)
    assert (out.float() - ref).abs().max().item() <= TOL[dtype]
    other = attention_prefill(q, k, v, D, mask=mask, causal=causal, impl="mma")
    assert (out.float() - other.float()).abs().max().item() <= 2 * TOL[dtype]
    again = attention_prefill(q, k, v, D, mask=mask, causal=causal, impl="tc")
    assert torch.equal(out, again)
    torch.cuda.synchronize()
    st = (ctypes.c_int * 4)()
    assert lib().eb_device_status(st, 0) == 0 and st[0] == 0, list(st)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,Sk,D,nsplit", [
    (2, 3, 128, 64, 1), (2, 3, 130, 64, 3), (16, 5, 640, 128, None), (3, 2, 1, 128, 1), (3, 2, 5, 64, 4),
    (8, 12, 2048, 128, None), (1, 1, 700, 128, 11),
])
def test_decode(B, H, Sk, D, nsplit, dtype):
    from energonai_b200.attention import attention_decode
    g = torch.Generator(device="cuda").manual_seed(Sk + D)
    max_len = Sk + 7
    cache = torch.randn(B, max_len, 3 * H * D, device="cuda", generator=g).to(dtype)
    k, v = cache[:, :, :H * D], cache[:, :, H * D:2 * H * D]
    q = cache[:, Sk - 1, 2 * H * D:]                       # the new token's query row inside the cache
    lens = [Sk] + [max(1, Sk // (i + 2)) for i in range(B - 1)]
    mask, _ = make_mask(B, Sk, lens, "left", dtype)
    mask_full = torch.zeros(B, max_len, device="cuda", dtype=dtype)
    mask_full[:, :Sk] = mask
    out = attention_decode(q, k, v, D, Sk, mask=mask_full, nsplit=nsplit)
    ref = reference(q.unsqueeze(1), k[:, :Sk], v[:, :Sk], D, mask, True)[:, 0]
    assert (out.float() - ref).abs().max().item() <= TOL[dtype]
    out2 = attention_decode(q, k, v, D, Sk, mask=mask_full, nsplit=nsplit)     # scratch is reusable, result deterministic
    assert torch.equal(out, out2)
    kv_dev = torch.tensor([Sk], dtype=torch.int32, device="cuda")
    out3 = attention_decode(q, k, v, D, max_len, mask=mask_full, nsplit=nsplit, kv_len_device=kv_dev)
    assert torch.equal(out, out3)


def test_decode_matches_last_prefill_row():
    from energonai_b200.attention import attention_prefill, attention_decode
    B, H, S, D = 4, 5, 300, 128
    qkv = torch.randn(B, S, 3 * H * D, device="cuda").half()
    k, v, q = qkv[:, :, :H * D], qkv[:, :, H * D:2 * H * D], qkv[:, :, 2 * H * D:]
    full = attention_prefill(q, k, v, D)
    last = attention_decode(q[:, -1], k, v, D, S)
    assert (full[:, -1].float() - last.float()).abs().max().item() <= 2e-3


def test_attention_rejects_unsupported():
    from energonai_b200.attention import attention_prefill
    q = torch.randn(1, 8, 96, device="cuda").half()
    with pytest.raises(RuntimeError, match="head_dim"):
        attention_prefill(q, q, q, 96, impl="mma")
    with pytest.raises(RuntimeError, match="head_dim"):
        attention_prefill(q, q, q, 96, impl="tc")
