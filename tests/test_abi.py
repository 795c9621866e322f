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
