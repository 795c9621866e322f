"""Small, self-contained launches of the hot kernels for profiler captures.

    python -m energonai_b200.profile_cases gemm_decode      # the four OPT-13B generation-step GEMM shapes
    python -m energonai_b200.profile_cases gemm_prefill     # one 8192-row prompt GEMM
    python -m energonai_b200.profile_cases attention        # prompt and generation-step attention

Each case holds a few hundred MB on the device (more than L2, so DRAM counters are
meaningful) and launches each kernel a handful of times.
"""
import sys

import torch


def gemm_decode():
    from .gemm import gemm
    h, f, M = 5120, 20480, 16
    for N, K in ((3 * h, h), (h, h), (f, h), (h, f)):
        w = torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02
        x = torch.randn(M, K, device="cuda", dtype=torch.float16)
        for _ in range(2):
            y = gemm(x, w, static_weight=True)
        torch.cuda.synchronize()
        print("gemm_decode", M, N, K, float((y.float() - x.float() @ w.float().t()).abs().max()))


def gemm_prefill():
    from .gemm import gemm
    M, N, K = 8192, 5120, 5120
    w = torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02
    x = torch.randn(M, K, device="cuda", dtype=torch.float16)
    for _ in range(3):
        y = gemm(x, w, static_weight=True)
    torch.cuda.synchronize()
    print("gemm_prefill", M, N, K, float((y.float() - x.float() @ w.float().t()).abs().max()))


def attention():
    from .attention import attention_prefill, attention_decode
    B, H, S, D = 16, 40, 512, 128
    cache = torch.randn(B, S + 128, 3 * H * D, device="cuda", dtype=torch.float16)
    k, v, q = cache[:, :, :H * D], cache[:, :, H * D:2 * H * D], cache[:, :, 2 * H * D:]
    for _ in range(2):
        o = attention_prefill(q[:, :S], k[:, :S], v[:, :S], D)
        o2 = attention_decode(q, k, v, D, S + 64, q_in_cache=True)
    torch.cuda.synchronize()
    print("attention", tuple(o.shape), tuple(o2.shape))


if __name__ == "__main__":
    {"gemm_decode": gemm_decode, "gemm_prefill": gemm_prefill, "attention": attention}[sys.argv[1]]()
