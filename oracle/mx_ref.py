"""ctypes view of the C restatement (oracle/mx_ref.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libmx_ref.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "mx_ref.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libmx_ref.so"])
    return _LIB


_REF_LIB = os.path.join(_HERE, "_ref", "libref_mxfp8_quant.so")
_ref_lib = None


def build_reference(reference_root: str, force: bool = False) -> str:
    """Compiles the reference's own quantiser (csrc/mxfp8_quantization.cu, where it lies under `reference_root`)
    plus oracle/ref_quant_shim.cu into oracle/_ref/libref_mxfp8_quant.so.  Needs nvcc, not a GPU."""
    src = os.path.join(reference_root, "csrc", "mxfp8_quantization.cu")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    if force and os.path.exists(_REF_LIB):
        os.remove(_REF_LIB)
    subprocess.check_call(["make", "-s", "-C", _HERE, "reference", f"REFERENCE={os.path.abspath(reference_root)}"])
    return _REF_LIB


def reference_quantizer():
    """ctypes handle of the reference's quantiser built by build_reference(), or None if it was not built.
    Entry points (device pointers): ref_quantize_to_mxfp8_bf16(out_i8, scales_f32, in_bf16, M, N, row_major, stream),
    ref_dequantize_from_mxfp8_bf16(out_bf16, in_i8, scales_f32, M, N, row_major, stream); both return the CUDA
    error code of the launch."""
    global _ref_lib
    if _ref_lib is None and os.path.exists(_REF_LIB):
        L = ctypes.CDLL(_REF_LIB)
        p, i32 = ctypes.c_void_p, ctypes.c_int
        L.ref_quantize_to_mxfp8_bf16.argtypes = [p, p, p, i32, i32, i32, p]
        L.ref_dequantize_from_mxfp8_bf16.argtypes = [p, p, p, i32, i32, i32, p]
        _ref_lib = L
    return _ref_lib


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB)
        p, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.mx_ref_num_threads.restype = i32
        L.mx_ref_quantize_rowwise.argtypes = [p, i64, i64, i32, p, p]
        L.mx_ref_quantize_colwise.argtypes = [p, i64, i64, i32, i32, p, p]
        L.mx_ref_dequantize.argtypes = [p, p, i64, i64, p]
        L.mx_ref_gemm.argtypes = [p, p, p, p, i64, i64, i64, f32, f32, p, p]
        L.mx_ref_gemm.restype = i32
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def num_threads() -> int:
    return int(lib().mx_ref_num_threads())


def quantize_rowwise(bits: np.ndarray, rule: int = 0):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    r, c = bits.shape
    codes = np.empty((r, c), np.uint8)
    scales = np.empty((r, (c + 31) // 32), np.uint8)
    lib().mx_ref_quantize_rowwise(_ptr(bits), r, c, rule, _ptr(codes), _ptr(scales))
    return codes, scales


def quantize_colwise(bits: np.ndarray, rule: int = 0, transpose_out: bool = True):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    r, c = bits.shape
    codes = np.empty((c, r) if transpose_out else (r, c), np.uint8)
    scales = np.empty((c, (r + 31) // 32), np.uint8)
    lib().mx_ref_quantize_colwise(_ptr(bits), r, c, rule, int(transpose_out), _ptr(codes), _ptr(scales))
    return codes, scales


def dequantize(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    r, c = codes.shape
    out = np.empty((r, c), np.float32)
    lib().mx_ref_dequantize(_ptr(codes), _ptr(scales), r, c, _ptr(out))
    return out


def gemm(a_codes, a_scales, b_codes, b_scales, alpha=1.0, beta=0.0, d_bits=None, bias_bits=None):
    a_codes = np.ascontiguousarray(a_codes, np.uint8); b_codes = np.ascontiguousarray(b_codes, np.uint8)
    a_scales = np.ascontiguousarray(a_scales, np.uint8); b_scales = np.ascontiguousarray(b_scales, np.uint8)
    m, k = a_codes.shape
    n = b_codes.shape[0]
    d = np.zeros((m, n), np.uint16) if d_bits is None else np.ascontiguousarray(d_bits, np.uint16).copy()
    bias = None if bias_bits is None else np.ascontiguousarray(bias_bits, np.uint16)
    rc = lib().mx_ref_gemm(_ptr(a_codes), _ptr(a_scales), _ptr(b_codes), _ptr(b_scales), m, n, k,
                           float(alpha), float(beta), _ptr(d), None if bias is None else _ptr(bias))
    if rc != 0:
        raise MemoryError("mx_ref_gemm: allocation failed")
    return d
