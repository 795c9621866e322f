"""GPU parity of the memory-bound kernels (padding offsets, (un)padding copies, head
transposes, scale_mask_softmax, LayerNorm) against the NumPy oracle, through the public
kernel API (which calls the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import kernels_np as K

pytestmark = pytest.mark.gpu

SEQ_LENS = [24, 127, 31, 65, 24, 127, 31, 65]     # reference fixture, tests/test_kernel/test_ft_transpose_pad.py:6
DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host(t):
    return t.float().cpu().numpy() if t.dtype == torch.bfloat16 else t.cpu().numpy()


def bits(t):
    """Bit pattern of a tensor for exact comparison (copies must be bit-exact)."""
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32).cpu().numpy()


CASES = [
    (SEQ_LENS, 128, 12, 64),                 # reference fixture
    ([5, 0, 3], 5, 2, 8),                    # empty sequence, a full one
    ([1], 1, 1, 1),                          # degenerate sizes, scalar path
    ([0, 0], 4, 3, 16),                      # nothing valid
    ([7, 2, 9, 9, 1], 9, 5, 6),              # head dim not a multiple of 8 -> scalar path for 16-bit types
    ([300, 17, 512, 1], 512, 16, 64),        # BERT-large shaped heads
]


@pytest.mark.parametrize("lens,S,H,D", CASES)
def test_build_padding_offsets_bit_exact(lens, S, H, D):
    from energonai_b200.kernel import ft_build_padding_offsets
    B = len(lens)
    valid_ref, off_ref = K.build_padding_offsets(lens, B, S)
    valid = torch.full((1,), -7, dtype=torch.int32).cuda()
    tmp = torch.full((B, S), -7, dtype=torch.int32).cuda()
    ft_build_padding_offsets(dev(np.array(lens, np.int32)), B, S, valid, tmp)
    assert int(valid.item()) == valid_ref
    got = tmp.view(-1).cpu().numpy()
    assert np.array_equal(got[:valid_ref], off_ref)
    assert np.all(got[valid_ref:] == -7)          # nothing beyond the valid count is written


def test_build_padding_offsets_known_answer():
    from energonai_b200.kernel import ft_build_padding_offsets
    valid = torch.zeros(1, dtype=torch.int32).cuda()
    tmp = torch.zeros(8, 128, dtype=torch.int32).cuda()
    ft_build_padding_offsets(dev(np.array(SEQ_LENS, np.int32)), 8, 128, valid, tmp)
    assert valid.item() == 494
    starts = np.concatenate([[0], np.cumsum(SEQ_LENS)[:-1]])
    assert tmp.view(-1)[torch.from_numpy(starts).cuda()].tolist() == [0, 104, 105, 202, 265, 369, 370, 467]


def test_build_padding_offsets_large_batch():
    from energonai_b200.kernel import ft_build_padding_offsets
    rng = np.random.default_rng(5)
    B, S = 3000, 40
    lens = rng.integers(0, S + 1, B).astype(np.int32)
    valid_ref, off_ref = K.build_padding_offsets(lens, B, S)
    valid = torch.zeros(1, dtype=torch.int32).cuda()
    tmp = torch.zeros(B * S, dtype=torch.int32).cuda()
    ft_build_padding_offsets(dev(lens), B, S, valid, tmp)
    assert valid.item() == valid_ref
    assert np.array_equal(tmp.cpu().numpy()[:valid_ref], off_ref)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("lens,S,H,D", CASES)
def test_ft_pipeline_bit_exact(lens, S, H, D, dt):
    """build -> remove -> transpose_rebuild -> transpose_remove -> rebuild, the sequence the
    reference's fixture test runs (tests/test_kernel/test_ft_transpose_pad.py:14-50), with
    every stage compared bit-for-bit against the oracle."""
    from energonai_b200 import kernel as EK
    B, n = len(lens), H * D
    rng = np.random.default_rng(10)
    tdt = DT[dt]
    x = dev(rng.standard_normal((3, B, S, n)).astype(np.float32), tdt)
    xn = [t.cpu() for t in x]
    valid_t = torch.zeros(1, dtype=torch.int32).cuda()
    tmp = torch.zeros(B, S, dtype=torch.int32).cuda()
    moff = torch.full((B, S), -1, dtype=torch.int32).cuda()
    EK.ft_build_padding_offsets(dev(np.array(lens, np.int32)), B, S, valid_t, tmp)
    valid = int(valid_t.item())
    _, off_ref = K.build_padding_offsets(lens, B, S)
    packed = [EK.ft_remove_padding(x[i], tmp, moff, valid, n) for i in range(3)]
    assert np.array_equal(moff.view(-1).cpu().numpy()[:valid], off_ref)
    refs = []
    for i in range(3):
        ref_i, _ = K.remove_padding(bits(xn[i]).reshape(B * S, n), off_ref, valid)
        refs.append(ref_i)
        assert packed[i].shape == (1, valid, n)
        assert np.array_equal(bits(packed[i]).reshape(valid, n), ref_i)
    bufs = [torch.zeros(B, H, S, D, dtype=tdt).cuda() for _ in range(3)]
    EK.ft_transpose_rebuild_padding(packed[0].view(1, valid, H, D), packed[1].view(1, valid, H, D),
                                    packed[2].view(1, valid, H, D), *bufs, B, S, H, D, valid, moff)
    for i in range(3):
        ref_buf = np.zeros((B, H, S, D), refs[i].dtype)
        K.transpose_rebuild_padding(refs[i], ref_buf, B, S, H, D, valid, off_ref)
        assert np.array_equal(bits(bufs[i]), ref_buf)
    back = EK.ft_transpose_remove_padding(bufs[2], valid, B, S, H, D, moff)
    assert back.shape == (1, valid, n)
    assert np.array_equal(bits(back).reshape(valid, n), refs[2])
    rebuilt = EK.ft_rebuild_padding(back, moff, valid, n, B, S)
    assert np.array_equal(bits(rebuilt), K.rebuild_padding(refs[2], off_ref, valid, B, S))


def test_transpose_rebuild_leaves_padding_rows_untouched():
    from energonai_b200 import kernel as EK
    lens, S, H, D = [3, 1], 4, 2, 8
    B = 2
    valid, off = K.build_padding_offsets(lens, B, S)
    q = torch.randn(valid, H, D).cuda()
    bufs = [torch.full((B, H, S, D), 9.0).cuda() for _ in range(3)]
    EK.ft_transpose_rebuild_padding(q, q, q, *bufs, B, S, H, D, valid, dev(off))
    ref = np.full((B, H, S, D), 9.0, np.float32)
    K.transpose_rebuild_padding(q.cpu().numpy(), ref, B, S, H, D, valid, off)
    for b_ in bufs:
        assert np.array_equal(b_.cpu().numpy(), ref)


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("lens,S,H,D", CASES + [(SEQ_LENS, 128, 12, 192)])   # 3*head_dim, as examples/gpt/gpt.py:103 calls it
def test_turbo_transposes_bit_exact(lens, S, H, D, dt):
    from energonai_b200.kernel import transpose_pad, transpose_depad
    B, tot = len(lens), int(sum(lens))
    rng = np.random.default_rng(11)
    packed = dev(rng.standard_normal((1, tot, H, D)).astype(np.float32), DT[dt])
    padded = transpose_pad(packed, B, S, dev(np.array(lens, np.int64)), H, D)     # int64 lens as the reference's test passes
    ref = K.transpose_pad(bits(packed), B, S, lens, H, D)
    assert padded.shape == (B, H, S, D)
    assert np.array_equal(bits(padded), ref)
    sum_seq = tot + 2                                                                # rows past the total are zeroed
    depad = transpose_depad(padded, B, sum_seq, S, dev(np.array(lens, np.int32)), H, D)
    assert depad.shape == (1, sum_seq, H, D)
    assert np.array_equal(bits(depad), K.transpose_depad(ref, B, sum_seq, S, lens, H, D))
    assert np.array_equal(bits(depad)[0, :tot], bits(packed)[0])


def test_turbo_identity_of_reference_test():
    """tests/test_kernel/test_transpose_pad_fusion_kernel.py:63-79."""
    from energonai_b200.kernel import transpose_pad, transpose_depad, depad
    B, S, H, D = 8, 128, 12, 64
    hs = torch.zeros(B, S, H * D)
    for b, L in enumerate(SEQ_LENS):
        hs[b, :L] = torch.randn(L, H * D)
    hs = hs.cuda()
    lens = torch.tensor(SEQ_LENS, dtype=torch.int64).cuda()
    res_original_pad = hs.view(B, S, H, D).permute(0, 2, 1, 3)
    input_depad = depad(hs, B, SEQ_LENS).view(1, -1, H, D)
    assert torch.equal(transpose_pad(input_depad, B, S, lens, H, D), res_original_pad)
    assert torch.equal(transpose_depad(res_original_pad, B, sum(SEQ_LENS), S, lens, H, D), input_depad)


SOFTMAX_CASES = [(2, 3, 8), (3, 2, 33), (2, 2, 128), (1, 2, 512), (1, 1, 1024), (1, 1, 1500), (1, 1, 2304), (2, 1, 1)]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("B,H,S", SOFTMAX_CASES)
def test_scale_mask_softmax(B, H, S, dt):
    from energonai_b200.kernel import scale_mask_softmax
    rng = np.random.default_rng(S)
    tdt = DT[dt]
    x = dev((rng.standard_normal((B, H, S, S)) * 3).astype(np.float32), tdt)
    lens = rng.integers(0, S + 1, B).astype(np.int32)
    lens[0] = S
    x_in = host(x)
    out = scale_mask_softmax(B, S, H, x, dev(lens))
    assert out.data_ptr() == x.data_ptr()
    got = host(out).astype(np.float32)
    ref = K.scale_mask_softmax(x_in.astype(np.float32), lens, B, S, H)
    tol = {"f32": 2e-6, "f16": 1e-3, "bf16": 8e-3}[dt]                 # output rounding of a probability <= 1
    for b in range(B):
        L = int(lens[b])
        assert np.array_equal(got[b, :, L:], x_in[b, :, L:].astype(np.float32))     # untouched rows, bit-exact
        assert np.abs(got[b, :, :L] - ref[b, :, :L]).max(initial=0) <= tol
        iu = np.triu_indices(S, 1)
        assert not got[b][:, :L][:, iu[0][iu[0] < L], iu[1][iu[0] < L]].any()        # masked keys are exactly 0


def test_scale_mask_softmax_extension_flags():
    from energonai_b200.kernel import scale_mask_softmax
    from energonai_b200._lib import SM_KEYLEN, SM_ALLROWS
    B, H, S = 2, 2, 40
    rng = np.random.default_rng(0)
    x = rng.standard_normal((B, H, S, S)).astype(np.float32)
    lens = np.array([40, 13], np.int32)
    out = scale_mask_softmax(B, S, H, dev(x), dev(lens), flags=SM_KEYLEN | SM_ALLROWS, scale=0.125).cpu().numpy()
    for b in range(B):
        L = lens[b]
        e = np.exp((x[b, :, :, :L] * 0.125).astype(np.float64))
        assert np.allclose(out[b, :, :, :L], e / e.sum(-1, keepdims=True), atol=2e-6)
        assert not out[b, :, :, L:].any()


LN_CASES = [(7, 768), (5, 1024), (16, 5120), (3, 9216), (4, 12288), (3, 20480), (2, 50), (3, 7), (1, 1), (33, 4104)]


@pytest.mark.parametrize("din,dout", [("f32", "f32"), ("f16", "f16"), ("bf16", "bf16"), ("f32", "f16"), ("f16", "f32")])
@pytest.mark.parametrize("n1,n2", LN_CASES)
def test_layer_norm(n1, n2, din, dout):
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    rng = np.random.default_rng(n2)
    x = dev((rng.standard_normal((n1, n2)) * 2 + 0.5).astype(np.float32), DT[din])
    g = dev((1 + 0.2 * rng.standard_normal(n2)).astype(np.float32), DT[dout])
    bt = dev((0.2 * rng.standard_normal(n2)).astype(np.float32), DT[dout])
    y, mean, invvar = layer_norm_forward(x, g, bt, 1e-5, return_stats=True)
    ref_y, ref_mu, ref_iv = K.layer_norm_fwd(host(x).astype(np.float64), host(g).astype(np.float64),
                                             host(bt).astype(np.float64), 1e-5)
    tol = {"f32": 2e-5, "f16": 4e-3, "bf16": 3e-2}[dout]               # one rounding of |y| <= ~8 in the output type
    assert y.dtype == DT[dout]
    assert np.abs(host(y).astype(np.float64) - ref_y).max() <= tol
    assert np.allclose(mean.cpu().numpy(), ref_mu, atol=1e-5)
    assert np.allclose(invvar.cpu().numpy(), ref_iv, rtol=1e-4)


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("n1,n2", [(6, 5120), (3, 50), (5, 1024)])
def test_layer_norm_fused_residual_bias(n1, n2, dt):
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    rng = np.random.default_rng(1)
    tdt = DT[dt]
    x, r = (dev(rng.standard_normal((n1, n2)).astype(np.float32), tdt) for _ in range(2))
    ab = dev(rng.standard_normal(n2).astype(np.float32), tdt)
    g, bt = dev(np.ones(n2, np.float32), tdt), dev(np.zeros(n2, np.float32), tdt)
    y, total = layer_norm_forward(x, g, bt, 1e-5, residual=r, add_bias=ab, return_sum=True)
    t_ref = (x.float() + r.float() + ab.float()).to(tdt)
    assert torch.equal(total, t_ref) or (total.float() - t_ref.float()).abs().max() <= (1e-6 if dt == "f32" else 4e-2)
    ref_y, _, _ = K.layer_norm_fwd(host(total).astype(np.float64), None, None, 1e-5)
    tol = {"f32": 2e-5, "f16": 4e-3, "bf16": 3e-2}[dt]
    assert np.abs(host(y).astype(np.float64) - ref_y).max() <= tol


def test_layer_norm_module_matches_reference_interface():
    from energonai_b200.kernel import LayerNorm
    ln = LayerNorm(256, eps=1e-5, dtype=torch.float16).cuda()
    assert sorted(n for n, _ in ln.named_parameters()) == ["bias", "weight"]
    x = torch.randn(2, 9, 256, dtype=torch.float16).cuda()
    with torch.inference_mode():
        y = ln(x)
    ref = torch.nn.functional.layer_norm(x.float(), (256,), ln.weight.float(), ln.bias.float(), 1e-5)
    assert (y.float() - ref).abs().max() < 4e-3
    with pytest.raises(RuntimeError):
        ln(torch.randn(2, 9, 255, dtype=torch.float16).cuda())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,V,h,split", [(16, 50272, 5120, False), (3, 1001, 96, False), (5, 4096, 256, True), (1, 7, 8, False)])
def test_greedy_step_tail(B, V, h, split, dtype):
    """eb_greedy_step against the framework's arg-max / index / embedding sequence
    (energonai/model/model_factory.py:124-131, embedding.py:44-57): tokens, the written column, the
    next step's embedding (bit-exact: one rounded sum of the same two table rows) and the advanced
    position scalars; with the vocabulary split in two, the halves' outputs add up to the whole."""
    from energonai_b200.step import greedy_step
    g = torch.Generator(device="cuda").manual_seed(V + h)
    logits = torch.randn(B, V, device="cuda", generator=g).to(dtype)
    logits[0, V // 2] = logits[0, V - 1] = 50.0                       # a tie: the lower index wins
    word = torch.randn(V, h, device="cuda", generator=g).to(dtype)
    posw = torch.randn(40, h, device="cuda", generator=g).to(dtype)
    cols, pos = 12, 8
    out_ids = torch.full((B, cols), -1, dtype=torch.int64, device="cuda")
    tok = torch.empty(B, dtype=torch.int64, device="cuda")
    kv = torch.tensor([pos, pos + 1], dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    want_tok = logits.float().argmax(-1)
    assert want_tok[0].item() == V // 2
    want_hidden = (word[want_tok].float() + posw[pos + 1].float()).to(dtype)
    if not split:
        hidden = torch.empty(B, 1, h, dtype=dtype, device="cuda")
        greedy_step(logits, out_ids, tok, kv, counter, word_emb=word, pos_emb=posw, hidden_out=hidden.view(B, h))
        assert torch.equal(hidden.view(B, h), want_hidden)
    else:
        half = V // 2
        parts = []
        for r in range(2):
            kv_r = torch.tensor([pos, pos + 1], dtype=torch.int32, device="cuda")
            hidden = torch.empty(B, h, dtype=dtype, device="cuda")
            greedy_step(logits, out_ids, tok, kv_r if r else kv, counter, word_emb=word[r * half:(r + 1) * half].contiguous(),
                        pos_emb=posw, hidden_out=hidden, vocab_start=r * half, add_pos=(r == 0))
            parts.append(hidden.float())
        assert torch.equal((parts[0] + parts[1]).to(dtype), want_hidden)
    assert torch.equal(tok, want_tok)
    assert torch.equal(out_ids[:, pos + 1], want_tok) and (out_ids[:, :pos + 1] == -1).all() and (out_ids[:, pos + 2:] == -1).all()
    assert kv.tolist() == [pos + 1, pos + 2] and counter.item() == 0
    if not split and dtype != torch.float32:
        # fp32 logits (what the LM head of a generation step produces) beside 16-bit tables
        hidden2 = torch.empty(B, h, dtype=dtype, device="cuda")
        kv2 = torch.tensor([pos, pos + 1], dtype=torch.int32, device="cuda")
        greedy_step(logits.float(), out_ids, tok, kv2, counter, word_emb=word, pos_emb=posw, hidden_out=hidden2)
        assert torch.equal(tok, want_tok) and torch.equal(hidden2, want_hidden)
    # a column outside the output is not written, and nothing else breaks
    kv.copy_(torch.tensor([pos, cols], dtype=torch.int32))
    before = out_ids.clone()
    greedy_step(logits, out_ids, tok, kv, counter)
    assert torch.equal(out_ids, before) and kv.tolist() == [pos + 1, cols + 1]
