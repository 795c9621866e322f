"""The library's kernels against the REFERENCE'S OWN CUDA kernels on the same GPU.

oracle/_ref/libenergon_ref.so holds the reference's unmodified scale_mask_softmax, LayerNorm
and padding / transpose kernels (energonai/kernel/cuda_native/csrc/*.cu) recompiled for sm_100a
(oracle/ref_cuda/build_ref.py).  The reference has no test of its own for scale_mask_softmax
and LayerNorm; this comparison is their pin.  Cases stay inside the reference's launch limits:
sequence length <= 1024 for the softmax (one thread per key), heads * head_dim <= 1024 (fp32) /
2048 (fp16) for the FT transposes, int32 lengths, fp32 / fp16 only (LayerNorm also bf16).

Tolerances: copies and index work bit-exact; softmax 2e-6 (fp32) / one fp16 rounding 1e-3
(both sides use the fast-math exponential); LayerNorm one step of the output type.
The last test times both sides per kernel and writes the table the profiles quote."""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libenergon_ref.so")
LENS = [24, 127, 31, 65, 24, 127, 31, 65]          # the reference's kernel-test fixture


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libenergon_ref.so was not built (python oracle/ref_cuda/build_ref.py)")
    return ctypes.CDLL(REF_LIB)


def p(t):
    return ctypes.c_void_p(t.data_ptr())


def code(dtype):
    return {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("B,H,S", [(8, 12, 128), (3, 5, 77), (2, 4, 1024), (4, 16, 512), (1, 1, 1)])
def test_scale_mask_softmax_against_the_reference_kernel(ref, B, H, S, dtype):
    from energonai_b200.kernel import scale_mask_softmax
    g = torch.Generator(device="cuda").manual_seed(B * 31 + S)
    x = (torch.randn(B, H, S, S, device="cuda", generator=g) * 3).to(dtype)
    lens = torch.randint(1, S + 1, (B,), device="cuda", generator=g, dtype=torch.int32)
    lens[0] = S
    theirs = x.clone()
    assert ref.ref_scale_mask_softmax(B, S, H, p(theirs), p(lens), code(dtype)) == 0
    ours = scale_mask_softmax(B, S, H, x.clone(), lens)
    torch.cuda.synchronize()
    tol = 2e-6 if dtype == torch.float32 else 1e-3
    assert float((ours.float() - theirs.float()).abs().max()) <= tol
    # rows at and beyond the real length are left as they were, by both; masked keys are exactly 0
    for b in range(B):
        n = int(lens[b])
        assert torch.equal(ours[b, :, n:], x[b, :, n:]) and torch.equal(theirs[b, :, n:], x[b, :, n:])
    upper = torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1)
    assert not ours[0][:, upper].any() and not theirs[0][:, upper].any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n1,n2", [(64, 768), (1000, 1024), (512, 5120), (17, 12288), (33, 264), (8, 9216)])
def test_layer_norm_against_the_reference_kernel(ref, n1, n2, dtype):
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    g = torch.Generator(device="cuda").manual_seed(n1 + n2)
    x = (torch.randn(n1, n2, device="cuda", generator=g) * 2 + 0.5).to(dtype)
    gamma = (1 + 0.1 * torch.randn(n2, device="cuda", generator=g)).to(dtype)
    beta = (0.1 * torch.randn(n2, device="cuda", generator=g)).to(dtype)
    y_ref = torch.empty_like(x)
    mean_ref, iv_ref = torch.empty(n1, device="cuda"), torch.empty(n1, device="cuda")
    assert ref.ref_layer_norm(p(y_ref), p(mean_ref), p(iv_ref), p(x), p(gamma), p(beta), ctypes.c_longlong(n1), n2,
                              ctypes.c_double(1e-5), code(dtype)) == 0
    y, mean, iv = layer_norm_forward(x, gamma, beta, 1e-5, return_stats=True)
    torch.cuda.synchronize()
    assert float((mean - mean_ref).abs().max()) <= 2e-5 * (1 + float(mean_ref.abs().max()))
    assert float(((iv - iv_ref) / iv_ref).abs().max()) <= 2e-5
    # both sides round the same fp32 value up to the last bits of the statistics: outputs may
    # differ by one step of the output type (2^-10 / 2^-7 of the next power of two for fp16 / bf16)
    step = {torch.float32: 4e-6, torch.float16: 2 ** -9, torch.bfloat16: 2 ** -6}[dtype]
    err = (y.float() - y_ref.float()).abs()
    assert bool((err <= step * y_ref.float().abs() + step / 4).all()), float(err.max())


def fixture(dtype, B=8, S=128, H=12, D=64, lens=LENS):
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, S, H * D, device="cuda", generator=g).to(dtype)
    return lens_t, x, int(sum(lens))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_padding_kernels_against_the_reference_kernels(ref, dtype):
    """The reference's own kernel-test fixture (tests/test_kernel/test_ft_transpose_pad.py:6-11)
    through both implementations, every output compared bit for bit."""
    from energonai_b200 import kernel as EK
    B, S, H, D = 8, 128, 12, 64
    lens, x, V = fixture(dtype)
    dc = code(dtype)
    valid_r = torch.zeros(1, dtype=torch.int32, device="cuda")
    tmp_r = torch.zeros(B * S, dtype=torch.int32, device="cuda")
    assert ref.ref_build_padding_offsets(p(lens), B, S, p(valid_r), p(tmp_r)) == 0
    valid_o = torch.zeros(1, dtype=torch.int32, device="cuda")
    tmp_o = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    EK.ft_build_padding_offsets(lens, B, S, valid_o, tmp_o)
    assert int(valid_r) == int(valid_o) == V == 494
    assert torch.equal(tmp_r[:V], tmp_o.view(-1)[:V])

    off_r = torch.zeros(B * S, dtype=torch.int32, device="cuda")
    packed_r = torch.zeros(V, H * D, device="cuda", dtype=dtype)
    assert ref.ref_remove_padding(p(x), p(packed_r), p(tmp_r), p(off_r), V, H * D, dc) == 0
    off_o = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    packed_o = EK.ft_remove_padding(x, tmp_o, off_o, V, H * D)
    assert torch.equal(packed_o.view(V, -1), packed_r) and torch.equal(off_o.view(-1)[:V], off_r[:V])

    rebuilt_r = torch.zeros(B, S, H * D, device="cuda", dtype=dtype)        # the reference's wrapper pre-zeroes
    assert ref.ref_rebuild_padding(p(packed_r), p(rebuilt_r), p(off_r), V, H * D, dc) == 0
    assert torch.equal(EK.ft_rebuild_padding(packed_o, off_o, V, H * D, B, S), rebuilt_r)

    q_r = [torch.zeros(B, H, S, D, device="cuda", dtype=dtype) for _ in range(3)]
    srcs = [packed_r, packed_r * 2, packed_r * 3]
    assert ref.ref_transpose_rebuild_padding(p(srcs[0]), p(srcs[1]), p(srcs[2]), p(q_r[0]), p(q_r[1]), p(q_r[2]), B, S, H, D, V,
                                             p(off_r), dc) == 0
    q_o = [torch.zeros(B, H, S, D, device="cuda", dtype=dtype) for _ in range(3)]
    EK.ft_transpose_rebuild_padding(*[s_.view(1, V, H, D) for s_ in srcs], *q_o, B, S, H, D, V, off_o)
    for a, b in zip(q_o, q_r):
        assert torch.equal(a, b)

    back_r = torch.zeros(V, H * D, device="cuda", dtype=dtype)
    assert ref.ref_transpose_remove_padding(p(q_r[0]), p(back_r), V, B, S, H, D, p(off_r), dc) == 0
    assert torch.equal(EK.ft_transpose_remove_padding(q_o[0], V, B, S, H, D, off_o).view(V, -1), back_r)

    # Turbo transposes: packed [1, V, H, D'] <-> [B, H, S, D'], zero fill at the pads
    for Dp in (D, 3 * D):
        src = torch.randn(1, V, H, Dp, device="cuda").to(dtype)
        pad_r = torch.empty(B, H, S, Dp, device="cuda", dtype=dtype)
        assert ref.ref_transpose_pad(p(src), B, S, p(lens), H, Dp, p(pad_r), dc) == 0
        pad_o = EK.transpose_pad(src, B, S, lens, H, Dp)
        assert torch.equal(pad_o, pad_r)
        dep_r = torch.empty(1, V, H, Dp, device="cuda", dtype=dtype)
        assert ref.ref_transpose_depad(p(pad_r), B, S, p(lens), H, Dp, p(dep_r), dc) == 0
        assert torch.equal(EK.transpose_depad(pad_o, B, V, S, lens, H, Dp), dep_r) and torch.equal(dep_r, src)
    torch.cuda.synchronize()


def test_speed_against_the_reference_kernels(ref):
    """Device time per launch (CUDA events around ten launches on distinct buffers larger than
    L2 in total) of the reference kernel and of the library's, at BASELINE configuration 2's
    shapes.  Written to ref_kernel_speedups.txt in the run's output folder when that folder exists."""
    from energonai_b200 import kernel as EK
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    rows = []

    def timed(fn, n=10):
        fn(0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    B, H, S = 32, 16, 512
    rng = np.random.default_rng(1)
    lens = torch.from_numpy(rng.integers(32, S + 1, B).astype(np.int32)).cuda()
    bufs = [torch.randn(B, H, S, S, device="cuda", dtype=torch.float16) for _ in range(4)]     # 4 x 268 MB
    t_ref = timed(lambda i: ref.ref_scale_mask_softmax(B, S, H, p(bufs[i % 4]), p(lens), 1), 8)
    t_our = timed(lambda i: EK.scale_mask_softmax(B, S, H, bufs[i % 4], lens), 8)
    rows.append(("scale_mask_softmax [32,16,512,512] fp16", t_ref, t_our))
    del bufs
    for n1, n2 in ((16384, 1024), (8192, 5120)):
        xs = [torch.randn(n1, n2, device="cuda", dtype=torch.float16) for _ in range(6)]
        ys = [torch.empty_like(x) for x in xs]
        g, b = torch.ones(n2, device="cuda", dtype=torch.float16), torch.zeros(n2, device="cuda", dtype=torch.float16)
        mu, iv = torch.empty(n1, device="cuda"), torch.empty(n1, device="cuda")
        t_ref = timed(lambda i: ref.ref_layer_norm(p(ys[i % 6]), p(mu), p(iv), p(xs[i % 6]), p(g), p(b), ctypes.c_longlong(n1), n2,
                                                   ctypes.c_double(1e-5), 1), 12)
        t_our = timed(lambda i: layer_norm_forward(xs[i % 6], g, b, 1e-5), 12)
        rows.append((f"layer_norm {n1} x {n2} fp16", t_ref, t_our))
        del xs, ys
    B, S, H, D = 256, 512, 16, 64
    lens = torch.from_numpy(rng.integers(32, S + 1, B).astype(np.int32)).cuda()
    V = int(lens.sum())
    valid, tmp, off = (torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(B, S, dtype=torch.int32, device="cuda"),
                       torch.zeros(B, S, dtype=torch.int32, device="cuda"))
    rows.append(("ft_build_padding_offsets B=256 S=512", timed(lambda i: ref.ref_build_padding_offsets(p(lens), B, S, p(valid), p(tmp))),
                 timed(lambda i: EK.ft_build_padding_offsets(lens, B, S, valid, tmp))))
    x = torch.randn(B, S, H * D, device="cuda", dtype=torch.float16)
    packed = torch.empty(V, H * D, device="cuda", dtype=torch.float16)
    rows.append(("ft_remove_padding", timed(lambda i: ref.ref_remove_padding(p(x), p(packed), p(tmp), p(off), V, H * D, 1)),
                 timed(lambda i: EK.ft_remove_padding(x, tmp, off, V, H * D))))
    out = torch.empty(B, S, H * D, device="cuda", dtype=torch.float16)

    def ref_rebuild(i):
        out.zero_()                                   # the reference's wrapper allocates with torch::zeros
        ref.ref_rebuild_padding(p(packed), p(out), p(off), V, H * D, 1)
    rows.append(("ft_rebuild_padding (+ zero fill)", timed(ref_rebuild), timed(lambda i: EK.ft_rebuild_padding(packed, off, V, H * D, B, S))))
    q = [torch.empty(B, H, S, D, device="cuda", dtype=torch.float16) for _ in range(3)]
    p4 = packed.view(1, V, H, D)

    def ref_trp(i):
        for t in q:
            t.zero_()                                 # caller-zeroed outputs (tests/test_kernel/test_ft_transpose_pad.py:36-40)
        ref.ref_transpose_rebuild_padding(p(packed), p(packed), p(packed), p(q[0]), p(q[1]), p(q[2]), B, S, H, D, V, p(off), 1)

    def our_trp(i):
        for t in q:
            t.zero_()
        EK.ft_transpose_rebuild_padding(p4, p4, p4, *q, B, S, H, D, V, off)
    rows.append(("ft_transpose_rebuild_padding (3 tensors, + zeroing)", timed(ref_trp), timed(our_trp)))
    rows.append(("ft_transpose_remove_padding", timed(lambda i: ref.ref_transpose_remove_padding(p(q[0]), p(packed), V, B, S, H, D, p(off), 1)),
                 timed(lambda i: EK.ft_transpose_remove_padding(q[0], V, B, S, H, D, off))))
    pad = torch.empty(B, H, S, D, device="cuda", dtype=torch.float16)
    rows.append(("transpose_pad", timed(lambda i: ref.ref_transpose_pad(p(p4), B, S, p(lens), H, D, p(pad), 1)),
                 timed(lambda i: EK.transpose_pad(p4, B, S, lens, H, D))))
    rows.append(("transpose_depad", timed(lambda i: ref.ref_transpose_depad(p(pad), B, S, p(lens), H, D, p(packed), 1)),
                 timed(lambda i: EK.transpose_depad(pad, B, V, S, lens, H, D))))
    lines = [f"{name}: reference kernel {a:.1f} us, this library {b:.1f} us, ratio {a / b:.2f}" for name, a, b in rows]
    print("\n".join(lines))
    out_dir = os.path.join(ROOT, "gpurun_out")
    if os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "ref_kernel_speedups.txt"), "w") as f:
            f.write("\n".join(lines) + "\n")
    assert all(b > 0 for _, _, b in rows)
