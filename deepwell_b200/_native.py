"""ctypes binding of the C ABI declared in include/dw_mxfp8.h.

The shared library is the product: there is no Python, PyTorch or CPU stand-in for any of
these calls.  If the library is missing or a call fails this module raises; it never
falls back (contrast src/deepwell/kernels/cutlass_bindings.py:181-192 of the reference,
which silently drops to torch.matmul).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libdw_mxfp8.so")

DW_OK = 0
DIR_ROW, DIR_COL_T, DIR_COL = 0, 1, 2
RULE_OCP_FLOOR, RULE_REF_CEIL = 0, 1
SF_FLAT, SF_TILED = 0, 1

DIRECTIONS = {"row": DIR_ROW, "col": DIR_COL_T, "col_t": DIR_COL_T, "col_inplace": DIR_COL}
RULES = {"ocp_floor": RULE_OCP_FLOOR, "ref_ceil": RULE_REF_CEIL}
LAYOUTS = {"flat": SF_FLAT, "tcgen05": SF_TILED, "tiled": SF_TILED}

ABI_SYMBOLS = (
    "dw_mxfp8_abi_version", "dw_mxfp8_device_supported", "dw_mxfp8_error_string", "dw_mxfp8_scale_bytes",
    "dw_mxfp8_quantize", "dw_mxfp8_quantize_both", "dw_mxfp8_dequantize", "dw_mxfp8_gemm",
    "dw_mxfp8_gemm_workspace", "dw_mxfp8_check_status", "dw_mxfp8_gemm_set_variant",
    "dw_mxfp8_gemm_set_timing_buffer", "dw_mxfp8_gemm_splitk_static", "dw_mxfp8_gemm_fused",
)

_lib = None


class NativeLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads libdw_mxfp8.so (once).  Raises NativeLibraryError if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m deepwell_b200._build` "
            "(nvcc, sm_100a).  There is no fallback path.")
    L = ctypes.CDLL(LIB_PATH)
    missing = [name for name in ABI_SYMBOLS if not hasattr(L, name)]
    if missing:
        raise NativeLibraryError(f"{LIB_PATH} is older than the sources (no {missing[0]}): rebuild it with "
                                 "`python deepwell_b200/_build.py`")
    p, i64, i32, f32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    L.dw_mxfp8_abi_version.restype = i32
    L.dw_mxfp8_device_supported.argtypes = [i32]
    L.dw_mxfp8_error_string.argtypes = [i32]
    L.dw_mxfp8_error_string.restype = ctypes.c_char_p
    L.dw_mxfp8_scale_bytes.argtypes = [i64, i64, i32]
    L.dw_mxfp8_scale_bytes.restype = sz
    L.dw_mxfp8_quantize.argtypes = [p, p, p, i64, i64, i32, i32, i32, p]
    L.dw_mxfp8_quantize_both.argtypes = [p, p, p, p, p, i64, i64, i32, i32, p]
    L.dw_mxfp8_dequantize.argtypes = [p, p, p, i64, i64, i32, p]
    L.dw_mxfp8_gemm.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, p, sz, p, p]
    L.dw_mxfp8_gemm_workspace.argtypes = [i64, i64, i64]
    L.dw_mxfp8_gemm_workspace.restype = sz
    L.dw_mxfp8_check_status.argtypes = [p, p]
    L.dw_mxfp8_gemm_set_variant.argtypes = [i32]
    L.dw_mxfp8_gemm_set_timing_buffer.argtypes = [p, sz]
    L.dw_mxfp8_gemm_fused.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, i32, p, p, i32, p, p]
    L.dw_mxfp8_gemm_splitk_static.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, i32, p, p]
    _lib = L
    return L


def check(code: int, what: str) -> None:
    if code != DW_OK:
        msg = load().dw_mxfp8_error_string(code).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {code})")


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be on CUDA")


def scale_bytes(rows: int, k: int, layout: int) -> int:
    return int(load().dw_mxfp8_scale_bytes(rows, k, layout))


def quantize(x: torch.Tensor, direction: int = DIR_ROW, rule: int = RULE_OCP_FLOOR,
             layout: int = SF_FLAT) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, cols] -> (codes float8_e4m3fn, scales uint8).  See dw_mxfp8_quantize."""
    _require_cuda(x, "input")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise RuntimeError("input must be a 2-D bfloat16 tensor")
    x = x.contiguous()
    rows, cols = x.shape
    op_rows, op_k = (rows, cols) if direction == DIR_ROW else (cols, rows)
    code_shape = (cols, rows) if direction == DIR_COL_T else (rows, cols)
    codes = torch.empty(code_shape, dtype=torch.uint8, device=x.device)
    nbytes = scale_bytes(op_rows, op_k, layout)
    scales = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(load().dw_mxfp8_quantize(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, cols,
                                       direction, rule, layout, _stream(x.device)), "dw_mxfp8_quantize")
    if layout == SF_FLAT:
        scales = scales.view(op_rows, (op_k + 31) // 32)
    return codes.view(torch.float8_e4m3fn), scales


def quantize_both(x: torch.Tensor, rule: int = RULE_OCP_FLOOR, layout: int = SF_TILED):
    """One read of x -> (codes_row, scales_row, codes_col_t, scales_col).  See dw_mxfp8_quantize_both."""
    _require_cuda(x, "input")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise RuntimeError("input must be a 2-D bfloat16 tensor")
    x = x.contiguous()
    rows, cols = x.shape
    dev = x.device
    cr = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
    ct = torch.empty((cols, rows), dtype=torch.uint8, device=dev)
    sr = torch.empty(scale_bytes(rows, cols, layout), dtype=torch.uint8, device=dev)
    sc = torch.empty(scale_bytes(cols, rows, layout), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(load().dw_mxfp8_quantize_both(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), ct.data_ptr(), sc.data_ptr(),
                                            rows, cols, rule, layout, _stream(dev)), "dw_mxfp8_quantize_both")
    if layout == SF_FLAT:
        sr = sr.view(rows, (cols + 31) // 32)
        sc = sc.view(cols, (rows + 31) // 32)
    return cr.view(torch.float8_e4m3fn), sr, ct.view(torch.float8_e4m3fn), sc


def dequantize(codes: torch.Tensor, scales: torch.Tensor, layout: int = SF_FLAT) -> torch.Tensor:
    _require_cuda(codes, "input")
    _require_cuda(scales, "scales")
    if codes.dim() != 2 or codes.element_size() != 1:
        raise RuntimeError("codes must be a 2-D one-byte tensor")
    codes = codes.contiguous()
    scales = scales.contiguous()
    rows, cols = codes.shape
    if scales.numel() < scale_bytes(rows, cols, layout):
        raise RuntimeError("scale buffer too small for this shape and layout")
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=codes.device)
    with torch.cuda.device(codes.device):
        check(load().dw_mxfp8_dequantize(codes.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, cols, layout,
                                         _stream(codes.device)), "dw_mxfp8_dequantize")
    return out


_status_words = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the GEMM kernel sets if one of its bounded waits expires."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
        _status_words[key] = w
    return w


def gemm(a_codes: torch.Tensor, a_sf: torch.Tensor, b_codes: torch.Tensor, b_sf: torch.Tensor,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, alpha: float = 1.0,
         beta: float = 0.0) -> torch.Tensor:
    """D[M,N] = alpha * A[M,K] . B[N,K]^T + beta * D + bias; operands as produced by quantize(..., SF_TILED)."""
    for t, n in ((a_codes, "A"), (b_codes, "B"), (a_sf, "A scales"), (b_sf, "B scales")):
        _require_cuda(t, n)
    if a_codes.dim() != 2 or b_codes.dim() != 2:
        raise RuntimeError("operands must be 2-D")
    M, K = a_codes.shape
    N, Kb = b_codes.shape
    if K != Kb:
        raise RuntimeError(f"contraction mismatch: A is [{M},{K}], B is [{N},{Kb}]")
    dev = a_codes.device
    if a_sf.numel() < scale_bytes(M, K, SF_TILED) or b_sf.numel() < scale_bytes(N, K, SF_TILED):
        raise RuntimeError("scale buffers must be in the tiled (tcgen05) layout")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous bfloat16 [M, N] tensor")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous()):
        raise RuntimeError("bias must be a contiguous bfloat16 [N] tensor")
    sw = status_word(dev)
    ws_bytes = int(load().dw_mxfp8_gemm_workspace(M, N, K))      # non-zero when the GEMM will split K
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
    with torch.cuda.device(dev):
        check(load().dw_mxfp8_gemm(a_codes.data_ptr(), a_sf.data_ptr(), b_codes.data_ptr(), b_sf.data_ptr(),
                                   out.data_ptr(), None if bias is None else bias.data_ptr(), M, N, K,
                                   float(alpha), float(beta), None if ws is None else ws.data_ptr(), ws_bytes,
                                   sw.data_ptr(), _stream(dev)), "dw_mxfp8_gemm")
    return out


ACTIVATIONS = {"none": 0, "relu": 1, "gelu": 2, "silu": 3}


def gemm_fused(a_codes: torch.Tensor, a_sf: torch.Tensor, b_codes: torch.Tensor, b_sf: torch.Tensor,
               bias: Optional[torch.Tensor] = None, activation: str = "none", quantize_out: bool = True,
               write_d: bool = True, alpha: float = 1.0, rule: int = RULE_OCP_FLOOR):
    """act(alpha * A . B^T + bias) -> (D bf16 or None, codes or None, tiled scales or None).  See dw_mxfp8_gemm_fused."""
    for t, n in ((a_codes, "A"), (b_codes, "B"), (a_sf, "A scales"), (b_sf, "B scales")):
        _require_cuda(t, n)
    M, K = a_codes.shape
    N, Kb = b_codes.shape
    if K != Kb:
        raise RuntimeError(f"contraction mismatch: A is [{M},{K}], B is [{N},{Kb}]")
    dev = a_codes.device
    d = torch.empty((M, N), dtype=torch.bfloat16, device=dev) if write_d else None
    codes = torch.empty((M, N), dtype=torch.uint8, device=dev) if quantize_out else None
    scales = torch.empty(scale_bytes(M, N, SF_TILED), dtype=torch.uint8, device=dev) if quantize_out else None
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous()):
        raise RuntimeError("bias must be a contiguous bfloat16 [N] tensor")
    sw = status_word(dev)
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(dev):
        check(load().dw_mxfp8_gemm_fused(a_codes.data_ptr(), a_sf.data_ptr(), b_codes.data_ptr(), b_sf.data_ptr(), ptr(d),
                                         ptr(bias), M, N, K, float(alpha), 0.0, ACTIVATIONS[activation], ptr(codes),
                                         ptr(scales), rule, sw.data_ptr(), _stream(dev)), "dw_mxfp8_gemm_fused")
    return d, (None if codes is None else codes.view(torch.float8_e4m3fn)), scales


def check_status(device=None) -> None:
    """Synchronises the current stream and raises if a kernel flagged an expired wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sw = status_word(dev)
    with torch.cuda.device(dev):
        rc = load().dw_mxfp8_check_status(sw.data_ptr(), _stream(dev))
    if rc != DW_OK:
        code = int(sw.item())
        sw.zero_()
        check(rc, f"GEMM kernel (status word {code & 0xFF}, CTA {code >> 8})")


def set_gemm_variant(v: int, group_m: int = 0, splits: int = 0) -> None:
    """Kernel variant (0 = automatic), raster band height and split-K count for later GEMMs."""
    check(load().dw_mxfp8_gemm_set_variant(int(v) | (int(group_m) << 8) | (int(splits) << 16)), "dw_mxfp8_gemm_set_variant")
