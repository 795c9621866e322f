"""Small, self-contained launches of the hot kernels: what the profiler captures under profiles/
were taken on, and CUDA-event timings of the kernels that are not part of the benchmark's step.

    python tests/kernel_cases.py gemm_decode      # the four OPT-13B generation-step GEMM shapes
    python tests/kernel_cases.py gemm_prefill     # one 8192-row prompt GEMM
    python tests/kernel_cases.py attention        # prompt (both kernels) and generation-step attention
    python tests/kernel_cases.py attention_speed  # TFLOP/s of the two prompt kernels over sequence lengths
    python tests/kernel_cases.py membound         # event-timed GB/s of the memory-bound kernels
    python tests/kernel_cases.py softmax          # scale_mask_softmax timed alone, back to back
    python tests/kernel_cases.py layernorm        # LayerNorm timed alone, back to back

Each case holds a few hundred MB on the device (more than L2, so DRAM counters are
meaningful) and launches each kernel a handful of times.  Not a test module (pytest does not
collect it).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def gemm_decode():
    from energonai_b200.gemm import gemm
    h, f, M = 5120, 20480, 16
    for N, K in ((3 * h, h), (h, h), (f, h), (h, f)):
        w = torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02
        x = torch.randn(M, K, device="cuda", dtype=torch.float16)
        for _ in range(2):
            y = gemm(x, w, static_weight=True)
        torch.cuda.synchronize()
        print("gemm_decode", M, N, K, float((y.float() - x.float() @ w.float().t()).abs().max()))
    # the same QKV shape with the LayerNorm in front of it folded in (eb_gemm_ln)
    from energonai_b200.gemm import fold_layernorm
    N, K = 3 * h, h
    w = torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02
    x = torch.randn(M, K, device="cuda", dtype=torch.float16)
    gamma = torch.ones(K, device="cuda", dtype=torch.float16)
    beta = torch.zeros(K, device="cuda", dtype=torch.float16)
    w_f, colsum, bias32 = fold_layernorm(w, None, gamma, beta)
    for _ in range(2):
        y = gemm(x, w_f, static_weight=True, ln_fold=(colsum, bias32, 1e-5))
    torch.cuda.synchronize()
    ref = torch.nn.functional.layer_norm(x.float(), (K,)) @ w.float().t()
    print("gemm_decode ln_fold", M, N, K, float((y.float() - ref).abs().max()))


def gemm_prefill():
    from energonai_b200.gemm import gemm
    M, N, K = 8192, 5120, 5120
    w = torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02
    x = torch.randn(M, K, device="cuda", dtype=torch.float16)
    for _ in range(3):
        y = gemm(x, w, static_weight=True)
    torch.cuda.synchronize()
    print("gemm_prefill", M, N, K, float((y.float() - x.float() @ w.float().t()).abs().max()))


def attention():
    from energonai_b200.attention import attention_prefill, attention_decode
    B, H, S, D = 16, 40, 512, 128
    cache = torch.randn(B, S + 128, 3 * H * D, device="cuda", dtype=torch.float16)
    k, v, q = cache[:, :, :H * D], cache[:, :, H * D:2 * H * D], cache[:, :, 2 * H * D:]
    for _ in range(2):
        o = attention_prefill(q[:, :S], k[:, :S], v[:, :S], D, impl="tc")
        o1 = attention_prefill(q[:, :S], k[:, :S], v[:, :S], D, impl="mma")
        o2 = attention_decode(q, k, v, D, S + 64, q_in_cache=True)
    torch.cuda.synchronize()
    print("attention", tuple(o.shape), tuple(o2.shape), "tc vs mma max diff", float((o.float() - o1.float()).abs().max()))


def attention_speed():
    """Causal prompt attention, fp16, head_dim 128 and 64: device time of 20 back-to-back launches
    of each kernel (inputs of 80 MB and more per launch), useful flops = 4 B H S^2 D / 2."""
    from energonai_b200.attention import attention_prefill
    for (B, H, S, D) in ((16, 40, 512, 128), (16, 40, 1024, 128), (4, 40, 2048, 128), (2, 40, 8192, 128), (16, 12, 512, 64),
                         (4, 12, 4096, 64)):
        qkv = torch.randn(B, S, 3 * H * D, device="cuda").half()
        k, v, q = qkv[:, :, :H * D], qkv[:, :, H * D:2 * H * D], qkv[:, :, 2 * H * D:]
        out = torch.empty(B, S, H * D, device="cuda", dtype=torch.float16)
        line = f"B {B:2d} H {H} S {S:4d} D {D:3d}:"
        for impl in ("mma", "tc"):
            for _ in range(3):
                attention_prefill(q, k, v, D, out=out, impl=impl)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                attention_prefill(q, k, v, D, out=out, impl=impl)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 20
            line += f"  {impl} {us:8.1f} us {2.0 * B * H * S * S * D / us / 1e6:6.1f} TFLOP/s"
        print(line)



def membound():
    """CUDA-event timings of the memory-bound kernels at benchmark shapes (configuration 2:
    batch 32 x 512, hidden 1024, 16 heads; configuration 3 prompt pass: 8192 x 5120), reported as
    algorithmic GB/s.  Inputs are larger than L2 or the L2 is flushed between repetitions."""
    import numpy as np
    from energonai_b200 import kernel as EK
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / reps

    def report(name, nbytes, ms):
        print(f"{name}: {ms * 1e3:.1f} us, {nbytes / 1e6:.1f} MB algorithmic, {nbytes / ms / 1e6:.0f} GB/s")

    # the copies run at 8x configuration 2's batch so that a launch lasts ~100 us and the
    # ~10 us of host launch latency inside the event bracket stops mattering
    B, S, H, D = 256, 512, 16, 64
    h = H * D
    rng = np.random.default_rng(1)
    lens = torch.from_numpy(rng.integers(32, S + 1, B).astype(np.int32)).cuda()
    V = int(lens.sum())
    valid = torch.zeros(1, dtype=torch.int32, device="cuda")
    tmp = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    moff = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    x = torch.randn(B, S, h, device="cuda", dtype=torch.float16)
    report("ft_build_padding_offsets B=256 S=512", 4 * B + 4 * V + 4,
           timed(lambda: EK.ft_build_padding_offsets(lens, B, S, valid, tmp)))
    report("ft_remove_padding", 2 * V * h * 2 + 8 * V, timed(lambda: EK.ft_remove_padding(x, tmp, moff, V, h)))
    packed = EK.ft_remove_padding(x, tmp, moff, V, h)
    report("ft_rebuild_padding (zero rows included)", (V + B * S) * h * 2 + 4 * V,
           timed(lambda: EK.ft_rebuild_padding(packed, moff, V, h, B, S)))
    bufs = [torch.zeros(B, H, S, D, device="cuda", dtype=torch.float16) for _ in range(3)]
    p4 = packed.view(1, V, H, D)
    report("ft_transpose_rebuild_padding (3 tensors)", 3 * 2 * V * h * 2 + 4 * V,
           timed(lambda: EK.ft_transpose_rebuild_padding(p4, p4, p4, *bufs, B, S, H, D, V, moff)))
    report("ft_transpose_remove_padding", 2 * V * h * 2 + 4 * V,
           timed(lambda: EK.ft_transpose_remove_padding(bufs[0], V, B, S, H, D, moff)))
    report("transpose_pad", (V + B * S) * h * 2, timed(lambda: EK.transpose_pad(p4, B, S, lens, H, D)))
    report("transpose_depad", 2 * V * h * 2, timed(lambda: EK.transpose_depad(bufs[0], B, V, S, lens, H, D)))
    del bufs, x, packed, p4
    B = 32
    lens = lens[:B].contiguous()
    V = int(lens.sum())
    scores = torch.randn(B, H, S, S, device="cuda", dtype=torch.float16)
    vis = int(sum(int(l) * (int(l) + 1) // 2 for l in lens.tolist()))
    report("scale_mask_softmax [32,16,512,512] fp16 (visible reads + row writes)", (vis + V * S) * H * 2,
           timed(lambda: EK.scale_mask_softmax(B, S, H, scores, lens)))
    # the BERT-style use of configuration 2: key-length mask only, every query row written
    from energonai_b200._lib import SM_ALLROWS, SM_KEYLEN
    report("scale_mask_softmax [32,16,512,512] fp16, key-length mask, all rows (visible reads + row writes)",
           (V + B * S) * S * H * 2,
           timed(lambda: EK.scale_mask_softmax(B, S, H, scores, lens, flags=SM_KEYLEN | SM_ALLROWS, scale=0.125)))
    for rows, n in ((B * S, 1024), (8192, 5120)):
        xx = torch.randn(rows, n, device="cuda", dtype=torch.float16)
        g, b = torch.ones(n, device="cuda", dtype=torch.float16), torch.zeros(n, device="cuda", dtype=torch.float16)
        report(f"layer_norm {rows} x {n} fp16", 2 * rows * n * 2, timed(lambda: layer_norm_forward(xx, g, b, 1e-5)))
        rr = torch.randn_like(xx)
        report(f"layer_norm + residual + bias + sum_out {rows} x {n}", 4 * rows * n * 2,
               timed(lambda: layer_norm_forward(xx, g, b, 1e-5, residual=rr, add_bias=b, return_sum=True)))


def softmax():
    """scale_mask_softmax at configuration 2's shape timed alone: eight distinct 268 MB score
    tensors (2.1 GB, far beyond L2) processed back to back between one pair of CUDA events, so
    neither host launch latency nor cache residency is in the figure."""
    import numpy as np
    from energonai_b200 import kernel as EK
    from energonai_b200._lib import SM_ALLROWS, SM_KEYLEN
    B, H, S = 32, 16, 512
    rng = np.random.default_rng(1)
    lens_h = rng.integers(32, S + 1, B).astype(np.int32)
    lens = torch.from_numpy(lens_h).cuda()
    V = int(lens_h.sum())
    vis = int(sum(int(n) * (int(n) + 1) // 2 for n in lens_h))
    bufs = [torch.randn(B, H, S, S, device="cuda", dtype=torch.float16) for _ in range(8)]
    cases = (("causal + length mask (the reference's mode)", {}, (vis + V * S) * H * 2),
             ("key-length mask, all rows", dict(flags=SM_KEYLEN | SM_ALLROWS, scale=0.125), (V + B * S) * S * H * 2))
    for name, kw, nbytes in cases:
        for b in bufs[:2]:
            EK.scale_mask_softmax(B, S, H, b, lens, **kw)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for b in bufs:
            EK.scale_mask_softmax(B, S, H, b, lens, **kw)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / len(bufs)
        print(f"scale_mask_softmax [32,16,512,512] fp16, {name}: {us:.1f} us per launch, {nbytes / 1e6:.1f} MB algorithmic, "
              f"{nbytes / us / 1e3:.0f} GB/s")


def layernorm():
    """LayerNorm forward timed alone: eight distinct inputs back to back between one pair of CUDA
    events (each set larger than L2), algorithmic bytes = read x + write y."""
    from energonai_b200.kernel.cuda_native.layer_norm import layer_norm_forward
    for rows, n in ((131072, 1024), (32768, 5120)):
        xs = [torch.randn(rows, n, device="cuda", dtype=torch.float16) for _ in range(8)]
        g, b = torch.ones(n, device="cuda", dtype=torch.float16), torch.zeros(n, device="cuda", dtype=torch.float16)
        for x in xs[:2]:
            layer_norm_forward(x, g, b, 1e-5)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for x in xs:
            layer_norm_forward(x, g, b, 1e-5)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / len(xs)
        nbytes = 2 * rows * n * 2
        print(f"layer_norm {rows} x {n} fp16: {us:.1f} us per launch, {nbytes / 1e6:.1f} MB algorithmic, {nbytes / us / 1e3:.0f} GB/s")
        del xs


if __name__ == "__main__":
    {"gemm_decode": gemm_decode, "gemm_prefill": gemm_prefill, "attention": attention, "attention_speed": attention_speed,
     "membound": membound, "softmax": softmax, "layernorm": layernorm}[sys.argv[1]]()
