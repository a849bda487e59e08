"""CPU tests of the drop-in boundary: the C-ABI library loads, exports every symbol the header
declares, and rejects bad arguments before touching a GPU."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def header_functions():
    text = open(os.path.join(ROOT, "include", "dw_mxfp8.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dw_mxfp8_\w+)\s*\(", text)))


def test_header_and_library_agree(native_lib):
    from deepwell_b200 import _native as nv
    names = header_functions()
    assert len(names) >= 11
    for n in names:
        assert hasattr(native_lib, n), f"{n} declared in include/dw_mxfp8.h but not exported"
    assert sorted(nv.ABI_SYMBOLS) == names
    assert native_lib.dw_mxfp8_abi_version() == 2


def test_scale_bytes(native_lib):
    from deepwell_b200 import _native as nv
    from oracle import mx_oracle as o
    for rows, k in [(1, 32), (128, 128), (129, 4096), (300, 1000), (16384, 14336)]:
        assert nv.scale_bytes(rows, k, nv.SF_FLAT) == rows * ((k + 31) // 32)
        assert nv.scale_bytes(rows, k, nv.SF_TILED) == o.sf_tiled_size(rows, (k + 31) // 32)
    assert nv.scale_bytes(0, 128, nv.SF_TILED) == 0


def test_bad_arguments_are_rejected_without_a_gpu(native_lib):
    L = native_lib
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert L.dw_mxfp8_quantize(p16, p16, p16, -1, 32, 0, 0, 0, None) == -1          # negative shape
    assert L.dw_mxfp8_quantize(p16, p16, p16, 4, 32, 7, 0, 0, None) == -1           # bad direction
    assert L.dw_mxfp8_quantize(p16, p16, p16, 4, 32, 0, 5, 0, None) == -1           # bad rule
    assert L.dw_mxfp8_quantize(p16, p16, p16, 4, 32, 0, 0, 9, None) == -1           # bad layout
    assert L.dw_mxfp8_quantize(None, p16, p16, 4, 32, 0, 0, 0, None) == -1          # null input
    assert L.dw_mxfp8_quantize(p16, p16, p16, 0, 32, 0, 0, 0, None) == 0            # empty: nothing to do
    assert L.dw_mxfp8_quantize(p16, p16, p16, 1 << 20, 1 << 20, 0, 0, 0, None) == -5  # over capacity
    assert L.dw_mxfp8_quantize_both(p16, None, None, None, None, 4, 32, 0, 0, None) == -1
    assert L.dw_mxfp8_dequantize(p16, p16, p16, 4, 32, 3, None) == -1
    assert L.dw_mxfp8_gemm(p16, p16, p16, p16, p16, None, 128, 128, 100, 1.0, 0.0, None, 0, None, None) == -1   # K % 32
    assert L.dw_mxfp8_gemm(p16 + 1, p16, p16, p16, p16, None, 128, 128, 128, 1.0, 0.0, None, 0, None, None) == -1  # alignment
    assert L.dw_mxfp8_gemm(None, p16, p16, p16, p16, None, 128, 128, 128, 1.0, 0.0, None, 0, None, None) == -1
    assert L.dw_mxfp8_gemm(p16, p16, p16, p16, p16, None, 0, 128, 128, 1.0, 0.0, None, 0, None, None) == 0        # empty
    assert L.dw_mxfp8_gemm_set_variant(99) == -1
    assert L.dw_mxfp8_gemm_set_variant(0) == 0
    assert L.dw_mxfp8_gemm_workspace(16384, 4096, 4096) == 0
    for code in (0, -1, -2, -3, -4, -5, -77):
        assert len(L.dw_mxfp8_error_string(code)) > 0


def test_wrong_architecture_is_reported_by_every_launcher(native_lib):
    """With the device query faked to compute capability 9.x every launching entry point returns DW_ERR_ARCH
    before it touches the device (so this runs without a GPU); argument errors still come first."""
    L = native_lib
    buf = ctypes.create_string_buffer(1 << 16)
    p16 = (ctypes.addressof(buf) + 15) & ~15
    assert L.dw_mxfp8_debug_fake_device(9, 132) == 0
    try:
        assert L.dw_mxfp8_quantize(p16, p16, p16, 32, 32, 0, 0, 0, None) == -2
        assert L.dw_mxfp8_quantize(p16, p16, p16, 32, 32, 1, 0, 1, None) == -2          # tile kernel path
        assert L.dw_mxfp8_quantize(p16, p16, p16, 3, 5, 2, 0, 0, None) == -2            # generic kernel path
        assert L.dw_mxfp8_quantize_both(p16, p16, p16, p16, p16, 32, 32, 0, 1, None) == -2
        assert L.dw_mxfp8_quantize_both_colsum(p16, p16, p16, p16, p16, 32, 32, 0, 1, p16, 0, p16, 1 << 12, None) == -2
        assert L.dw_mxfp8_dequantize(p16, p16, p16, 4, 32, 0, None) == -2
        assert L.dw_mxfp8_update_amax_history(p16, ctypes.c_void_p(p16), 4, 64, None) == -2
        gemm_args = (p16, p16, p16, p16, p16, None, 128, 128, 128, 1.0, 0.0)
        assert L.dw_mxfp8_gemm(*gemm_args, None, 0, None, None) == -2
        assert L.dw_mxfp8_gemm_planned(*gemm_args, None, 0, 3, None, None) == -2
        assert L.dw_mxfp8_gemm_fused(*gemm_args, 1, None, None, 0, None, None) == -2
        assert L.dw_mxfp8_gemm_splitk_static(*gemm_args, 2, None, None) == -2
        groups = (ctypes.c_int * 1)(0)
        assert L.dw_mxfp8_gemm_grouped(p16, p16, p16, p16, p16, ctypes.cast(groups, ctypes.c_void_p), 128, 128, 128, 1, 128, 1.0,
                                       None, None) == -2
        assert L.dw_mxfp8_selftest_bounded_wait(1000, p16, None) == -2
        # argument errors are still reported first
        assert L.dw_mxfp8_gemm(p16, p16, p16, p16, p16, None, 128, 128, 100, 1.0, 0.0, None, 0, None, None) == -1
        assert L.dw_mxfp8_gemm_planned(*gemm_args, None, 0, 77, None, None) == -1       # no such variant
        assert L.dw_mxfp8_selftest_bounded_wait(10 ** 9, p16, None) == -5                 # longer than a test may wait
        # the planner sizes workspaces for the (faked) SM count without a device
        assert L.dw_mxfp8_gemm_workspace_planned(1024, 768, 8192, 4 << 16) == 4 * 1024 * 768 * 4
        assert L.dw_mxfp8_gemm_workspace_planned(1024, 768, 8192, 1 << 16) == 0
    finally:
        assert L.dw_mxfp8_debug_fake_device(-1, 0) == 0


def test_per_device_bookkeeping_with_a_faked_device(native_lib):
    """The SM count the planner uses is the current device's, not the first device's: the split-K workspace of a
    small problem follows the faked SM count."""
    L = native_lib
    try:
        L.dw_mxfp8_debug_fake_device(10, 148)
        big = L.dw_mxfp8_gemm_workspace_planned(1024, 1024, 16384, 0)
        L.dw_mxfp8_debug_fake_device(10, 16)                 # a 16-SM part: the same problem fills it, no split
        small = L.dw_mxfp8_gemm_workspace_planned(1024, 1024, 16384, 0)
        assert big > 0 and small == 0
    finally:
        L.dw_mxfp8_debug_fake_device(-1, 0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from deepwell_b200 import _native as nv
    monkeypatch.setattr(nv, "_lib", None)
    monkeypatch.setattr(nv, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(nv.NativeLibraryError):
        nv.load()


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "deepwell_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("the oracle", ""), f"{f} refers to the oracle package"


def test_tensor_layer_loads_and_refuses_cpu_tensors(native_lib):
    """deepwell_b200._C (csrc/python_bindings.cpp) imports, exports the per-layer calls and has no CPU path."""
    import torch
    from deepwell_b200 import _native
    ext = _native.ext()
    for name in ("quantize", "quantize_both", "gemm", "linear_forward", "linear_backward"):
        assert callable(getattr(ext, name)), name
    x = torch.zeros(32, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        ext.quantize(x, _native.DIR_ROW, _native.RULE_OCP_FLOOR, _native.SF_FLAT)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        ext.quantize_both(x, _native.RULE_OCP_FLOOR, _native.SF_TILED)
    u8 = torch.zeros(32, 32, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        ext.gemm(u8, u8, u8, u8, None, None, 1.0, 0.0, torch.zeros(1, dtype=torch.int32))
