"""The allocation-free generation-step attention entry point against the regular one.

eb_attention_decode_noalloc serves hosts that cannot allocate device memory on the serving path
(fixed memory pools, a locked allocator, raw-pointer embeddings): its split-KV scratch is an
array built into the library.  It runs the same kernel as eb_attention_decode, so the outputs
must be identical bit for bit, on a first call (which sets the array up) and on a second call
(which finds the previous call's contents in it).  This file is collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, q, k, v, out, mask, B, H, D, kv_len, nsplit, extra=()):
    from energonai_b200._lib import dtype_code, stream_ptr
    return fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), mask.data_ptr(), q.stride(0), q.stride(1),
              k.stride(0), k.stride(1), v.stride(0), v.stride(1), out.stride(0), mask.stride(0), B, H, kv_len, None, D,
              D ** -0.5, dtype_code(q.dtype), nsplit, *extra, stream_ptr())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_noalloc_decode_matches_regular_entry_point(dtype):
    from energonai_b200 import _lib
    L = _lib.lib()
    B, H, D, kv_len, nsplit = 6, 5, 128, 300, 4
    for attempt in range(2):                                   # two calls in a row share the built-in array
        g = torch.Generator(device="cuda").manual_seed(10 + attempt)
        cache = torch.randn(B, kv_len + 9, 3 * H * D, device="cuda", generator=g).to(dtype)
        k, v, q = cache[:, :, :H * D], cache[:, :, H * D:2 * H * D], cache[:, :, 2 * H * D:]
        mask = torch.zeros(B, kv_len + 9, device="cuda", dtype=dtype)
        mask[1, :40] = -10000.0
        nbytes = L.eb_attention_decode_scratch_bytes(B, H, D, nsplit)
        scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        ref = torch.empty(B, H * D, device="cuda", dtype=dtype)
        out = torch.full_like(ref, float("nan"))
        rc = _call(L.eb_attention_decode, q, k, v, ref, mask, B, H, D, kv_len, nsplit,
                   extra=(scratch.data_ptr(), scratch.numel()))
        assert rc == 0, _lib.last_error()
        before = torch.cuda.memory_allocated()
        rc = _call(L.eb_attention_decode_noalloc, q, k, v, out, mask, B, H, D, kv_len, nsplit)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(out, ref), (out.float() - ref.float()).abs().max()


def test_noalloc_decode_rejects_oversized_requests():
    from energonai_b200 import _lib
    L = _lib.lib()
    B, H, D, nsplit = 64, 96, 128, 64                           # 64*96*64*130*4 bytes = 204 MB of partials
    assert L.eb_attention_decode_scratch_bytes(B, H, D, nsplit) > (8 << 20)
    x = torch.zeros(B, 8, 3 * H * D, device="cuda", dtype=torch.float16)
    out = torch.zeros(B, H * D, device="cuda", dtype=torch.float16)
    mask = torch.zeros(B, 8, device="cuda", dtype=torch.float16)
    rc = _call(L.eb_attention_decode_noalloc, x[:, :, 2 * H * D:], x[:, :, :H * D], x[:, :, H * D:2 * H * D], out, mask,
               B, H, D, 8, nsplit)
    assert rc == -5 and "8388608" in _lib.last_error()
