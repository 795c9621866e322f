"""The C-ABI library loads without a GPU and exports every symbol the header declares;
argument validation that happens before any CUDA call is exercised too."""
import ctypes
import os

import pytest

from energonai_b200 import _lib


def test_header_declares_the_expected_entry_points():
    decls = _lib.parse_header()
    for name in ("eb_version", "eb_last_error", "eb_build_padding_offsets", "eb_remove_padding", "eb_rebuild_padding",
                 "eb_transpose_rebuild_padding", "eb_transpose_remove_padding", "eb_transpose_pad", "eb_transpose_depad",
                 "eb_scale_mask_softmax", "eb_layer_norm_fwd"):
        assert name in decls


def test_library_exports_every_declared_symbol():
    assert os.path.exists(_lib.LIB_PATH), "build the library first: python -m energonai_b200.build"
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in _lib.parse_header():
        assert hasattr(handle, name), name
    assert _lib.lib().eb_version() >= 100


def test_argument_validation_needs_no_gpu():
    L = _lib.lib()
    assert L.eb_scale_mask_softmax(None, None, 1, 8, 1, 7, 1, 1.0, None) == -1
    assert "dtype" in _lib.last_error()
    assert L.eb_remove_padding(None, None, None, None, 4, 8, _lib.F16, None) == -1
    assert "null" in _lib.last_error()
    assert L.eb_rebuild_padding(None, None, None, 9, 8, 2, 4, _lib.F16, 1, None) == -1
    assert L.eb_layer_norm_fwd(None, None, None, None, None, None, None, None, None, 4, 8, 1e-5, 0, 0, None) == -1
    # empty problems are accepted without touching the device
    assert L.eb_remove_padding(None, None, None, None, 0, 8, _lib.F16, None) == 0
    assert L.eb_scale_mask_softmax(None, None, 0, 8, 1, 0, 1, 1.0, None) == 0


def test_cpu_tensors_are_rejected():
    import torch
    from energonai_b200.kernel import scale_mask_softmax
    with pytest.raises(RuntimeError):
        scale_mask_softmax(1, 4, 1, torch.zeros(1, 1, 4, 4), torch.tensor([4], dtype=torch.int32))


def test_chain_op_struct_matches_the_header(tmp_path):
    """The ctypes mirror of struct eb_chain_op has the size and field offsets a C compiler gives
    the declaration in the header (the header itself compiles as plain C)."""
    import shutil
    import subprocess
    from energonai_b200.chain import ChainOp
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    fields = [name for name, _ in ChainOp._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{_lib.HEADER}"', 'int main(void) {',
             '  printf("%zu\\n", sizeof(eb_chain_op));']
    lines += [f'  printf("%zu\\n", offsetof(eb_chain_op, {f}));' for f in fields]
    lines += ['  return 0;', '}']
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == ctypes.sizeof(ChainOp)
    for f, off in zip(fields, out[1:]):
        assert int(off) == getattr(ChainOp, f).offset, f


def test_new_entry_points_validate_before_any_cuda_call():
    L = _lib.lib()
    # eb_gemm_ln: the folded vectors are required, and only generation-step batches are served
    assert L.eb_gemm_ln(None, 8, None, 8, None, 8, None, None, 1e-5, None, 0, 4, 8, 8, _lib.F16, _lib.F16, 0, 0, 0, None, 0, 0,
                        None, 0, None) == -1
    assert "ln_colsum" in _lib.last_error()
    assert L.eb_decode_chain(None, 0, 16, _lib.F16, None, 0, None, None) == -1
    assert L.eb_decode_chain_workspace_bytes(None, 0, 16) == 0


def test_exchange_context_validates_before_any_cuda_call():
    """Wrong group sizes, undersized areas and null contexts are refused with a message; none of
    these calls reaches the CUDA runtime."""
    L = _lib.lib()
    out = ctypes.c_void_p()
    assert L.eb_comm_create(0, 0, 1 << 20, 0, None, ctypes.byref(out)) == -1 and "world" in _lib.last_error()
    assert L.eb_comm_create(3, 2, 1 << 20, 0, None, ctypes.byref(out)) == -1 and "rank" in _lib.last_error()
    assert L.eb_comm_create(0, 9, 1 << 20, 0, None, ctypes.byref(out)) == -1
    assert L.eb_comm_create(0, 2, 1000, 0, None, ctypes.byref(out)) == -1 and "512" in _lib.last_error()
    assert L.eb_comm_create(0, 2, 1 << 20, 100, None, ctypes.byref(out)) == -1 and "bulk" in _lib.last_error()
    assert L.eb_comm_create(0, 2, 1 << 20, 0, None, None) == -1
    assert L.eb_comm_area_bytes(1 << 20, 1 << 20) == 4096 + (2 << 20)
    assert L.eb_reduce_broadcast_stage_bytes(8, 8192, 5120) == 8 * 1024 * 5120 * 2
    assert L.eb_reduce_broadcast(None, 256, 64, _lib.F16, 0, 0, None, None, 0, None) == -1
    assert L.eb_gemm_reduce_scatter(None, 8, None, 8, 256, 64, 64, _lib.F16, 0, None, 0, None) == -1
    assert out.value is None
    assert L.eb_comm_handle_bytes() == 64
    assert L.eb_comm_exchange_bytes(8, 16, 5120) == 8 * 16 * 5120 * 4
    assert L.eb_comm_exchange_bytes(0, 16, 5120) == 0
    assert L.eb_allreduce(None, None, 8, _lib.F16, None) == -1 and "null context" in _lib.last_error()
    assert L.eb_comm_status(None, None, 0) == -1
    assert L.eb_comm_connect(None, None, 0) == -1
    assert L.eb_comm_destroy(None) == 0
    assert L.eb_gemm_allreduce(None, 8, None, 8, None, 8, None, None, 0, 4, 8, 8, _lib.F16, _lib.F16, 0, 0, 0, None, 0, 0, None,
                               0, None, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No CPU or PyTorch fallback: without the built library every kernel call raises."""
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libenergon_b200.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_generation_attention_split_rule():
    """Key splits of the generation-step attention: none below a thousand keys per CTA (measured
    to lose there), never more than one per 64-key tile or than three CTAs per SM need."""
    from energonai_b200.attention import pick_nsplit
    assert [pick_nsplit(16, h, 640) for h in (5, 10, 20, 40)] == [1, 1, 1, 1]
    assert pick_nsplit(1, 40, 8192) == 8
    assert pick_nsplit(2, 5, 4096) == 4
    assert pick_nsplit(8, 96, 2048) == 1          # 768 (sequence, head) pairs fill the machine already
    assert pick_nsplit(1, 1, 100) == 1
    assert pick_nsplit(1, 1, 1 << 20) == 64


def test_attention_and_step_tail_validate_before_any_cuda_call():
    L = _lib.lib()
    buf = ctypes.create_string_buffer(64)
    a = ctypes.addressof(buf) & ~15 or 16
    # tensor-core prompt attention: head_dim, dtype, strides, scale
    args = lambda **kw: [kw.get("q", a), a, a, a, None, 8, 8, 8, 8, 8, 8, 8, 8, 0, 1, 1, 8, 8, kw.get("d", 64),
                         kw.get("causal", 1), kw.get("scale", 0.125), kw.get("dtype", _lib.F16), None]
    assert L.eb_attention_prefill_tc(*args(d=96)) == -1 and "head_dim" in _lib.last_error()
    assert L.eb_attention_prefill_tc(*args(dtype=_lib.F32)) == -1 and "fp16 or bf16" in _lib.last_error()
    assert L.eb_attention_prefill_tc(*args(q=None)) == -1 and "null" in _lib.last_error()
    assert L.eb_attention_prefill_tc(*args(scale=0.0)) == -1 and "scale" in _lib.last_error()
    bad = args()
    bad[6] = 12                       # q row stride not a multiple of 8
    assert L.eb_attention_prefill_tc(*bad) == -1 and "strides" in _lib.last_error()
    # the tail of a generation step: sizes and pointers
    step = lambda **kw: [kw.get("logits", a), kw.get("ld", 16), kw.get("batch", 2), 16, kw.get("dtype", _lib.F16), a, 4, 4, None, a,
                         kw.get("word", None), 0, 0, None, 0, 1, 0, _lib.F16, None, 0, kw.get("counter", a), None]
    assert L.eb_greedy_step(*step(batch=0)) == 0
    assert L.eb_greedy_step(*step(dtype=9)) == -1 and "dtype" in _lib.last_error()
    assert L.eb_greedy_step(*step(logits=None)) == -1 and "null" in _lib.last_error()
    assert L.eb_greedy_step(*step(ld=8)) == -1 and "leading" in _lib.last_error()
    assert L.eb_greedy_step(*step(word=a)) == -1 and "embedding" in _lib.last_error()
