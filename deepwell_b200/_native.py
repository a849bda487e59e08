"""Binding of the C ABI declared in include/dw_mxfp8.h.

Two routes reach the same shared library.  ctypes (load()) exposes every entry point with raw
pointers: the tests and the rarely-called functions use it.  deepwell_b200._C (ext(), built from
csrc/python_bindings.cpp) wraps the per-layer calls (quantize, quantize_both, gemm, the linear
layer's forward and backward) so that one Python call allocates the outputs and launches; the
hot path of DWLinear goes through it because the ctypes route costs more host time than a small
layer's kernels take.

The shared library is the product: there is no Python, PyTorch or CPU stand-in for any of
these calls.  If the library or the extension is missing or a call fails this module raises; it
never falls back (contrast src/deepwell/kernels/cutlass_bindings.py:181-192 of the reference,
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
QUANT_OVERLAP_PREVIOUS = 1

DIRECTIONS = {"row": DIR_ROW, "col": DIR_COL_T, "col_t": DIR_COL_T, "col_inplace": DIR_COL}
RULES = {"ocp_floor": RULE_OCP_FLOOR, "ref_ceil": RULE_REF_CEIL}
LAYOUTS = {"flat": SF_FLAT, "tcgen05": SF_TILED, "tiled": SF_TILED}

ABI_SYMBOLS = (
    "dw_mxfp8_abi_version", "dw_mxfp8_device_supported", "dw_mxfp8_error_string", "dw_mxfp8_scale_bytes",
    "dw_mxfp8_quantize", "dw_mxfp8_quantize_both", "dw_mxfp8_dequantize", "dw_mxfp8_gemm",
    "dw_mxfp8_gemm_workspace", "dw_mxfp8_check_status", "dw_mxfp8_gemm_set_variant",
    "dw_mxfp8_gemm_set_timing_buffer", "dw_mxfp8_gemm_splitk_static", "dw_mxfp8_gemm_fused",
    "dw_mxfp8_colsum_workspace", "dw_mxfp8_quantize_both_colsum", "dw_mxfp8_gemm_grouped",
    "dw_mxfp8_update_amax_history", "dw_mxfp8_gemm_planned", "dw_mxfp8_gemm_workspace_planned",
    "dw_mxfp8_selftest_bounded_wait", "dw_mxfp8_debug_fake_device", "dw_mxfp8_debug_counter",
    "dw_mxfp8_quantize_set_tuning", "dw_mxfp8_quantize_ex", "dw_mxfp8_quantize_rows_batch",
    "dw_mxfp8_copy_2d_async",
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
    L.dw_mxfp8_quantize_set_tuning.argtypes = [i32]
    L.dw_mxfp8_quantize_ex.argtypes = [p, p, p, i64, i64, i32, i32, i32, i32, p]
    L.dw_mxfp8_quantize_rows_batch.argtypes = [i32, ctypes.POINTER(p), ctypes.POINTER(p), ctypes.POINTER(p),
                                               ctypes.POINTER(i64), ctypes.POINTER(i64), i32, i32, i32, p]
    L.dw_mxfp8_copy_2d_async.argtypes = [p, sz, p, sz, sz, sz, p]
    L.dw_mxfp8_quantize_both.argtypes = [p, p, p, p, p, i64, i64, i32, i32, p]
    L.dw_mxfp8_dequantize.argtypes = [p, p, p, i64, i64, i32, p]
    L.dw_mxfp8_update_amax_history.argtypes = [p, p, i32, i64, p]
    L.dw_mxfp8_colsum_workspace.argtypes = [i64, i64]
    L.dw_mxfp8_colsum_workspace.restype = sz
    L.dw_mxfp8_quantize_both_colsum.argtypes = [p, p, p, p, p, i64, i64, i32, i32, p, i32, p, sz, p]
    L.dw_mxfp8_gemm.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, p, sz, p, p]
    L.dw_mxfp8_gemm_workspace.argtypes = [i64, i64, i64]
    L.dw_mxfp8_gemm_workspace.restype = sz
    L.dw_mxfp8_check_status.argtypes = [p, p]
    L.dw_mxfp8_gemm_set_variant.argtypes = [i32]
    L.dw_mxfp8_gemm_set_timing_buffer.argtypes = [p, sz]
    L.dw_mxfp8_gemm_fused.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, i32, p, p, i32, p, p]
    L.dw_mxfp8_gemm_grouped.argtypes = [p, p, p, p, p, p, i64, i64, i64, i32, i32, f32, p, p]
    L.dw_mxfp8_gemm_splitk_static.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, i32, p, p]
    L.dw_mxfp8_gemm_planned.argtypes = [p, p, p, p, p, p, i64, i64, i64, f32, f32, p, sz, i32, p, p]
    L.dw_mxfp8_gemm_workspace_planned.argtypes = [i64, i64, i64, i32]
    L.dw_mxfp8_gemm_workspace_planned.restype = sz
    L.dw_mxfp8_selftest_bounded_wait.argtypes = [ctypes.c_longlong, p, p]
    L.dw_mxfp8_debug_fake_device.argtypes = [i32, i32]
    L.dw_mxfp8_debug_counter.argtypes = [i32]
    L.dw_mxfp8_debug_counter.restype = ctypes.c_longlong
    _lib = L
    return L


_ext = None


def ext():
    """The torch-tensor layer over the library (deepwell_b200._C).  Raises NativeLibraryError if it is not built."""
    global _ext
    if _ext is None:
        load()
        try:
            from . import _C
        except ImportError as e:
            raise NativeLibraryError(f"deepwell_b200/_C.so is missing or does not load ({e}): build it with "
                                     "`python deepwell_b200/_build.py`.  There is no fallback path.") from e
        _ext = _C
    return _ext


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
    return ext().quantize(x, direction, rule, layout)


def quantize_into(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, direction: int = DIR_ROW,
                  rule: int = RULE_OCP_FLOOR, layout: int = SF_TILED) -> None:
    """dw_mxfp8_quantize into caller-provided buffers (views into larger operands, e.g. one expert's slice of a
    stacked weight): codes and scales must be contiguous byte tensors of the right size."""
    _require_cuda(x, "input")
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise RuntimeError("input must be a contiguous 2-D bfloat16 tensor")
    rows, cols = x.shape
    op_rows, op_k = (rows, cols) if direction == DIR_ROW else (cols, rows)
    if codes.numel() * codes.element_size() != rows * cols or not codes.is_contiguous() or not scales.is_contiguous() \
            or scales.numel() < scale_bytes(op_rows, op_k, layout):
        raise RuntimeError("output buffers do not match the operand")
    with torch.cuda.device(x.device):
        check(load().dw_mxfp8_quantize(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, cols, direction, rule, layout,
                                       _stream(x.device)), "dw_mxfp8_quantize")


def copy_2d_async(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width_bytes: int, height: int, device) -> None:
    """dw_mxfp8_copy_2d_async on the current stream of `device`: `height` rows of `width_bytes` bytes between two device
    addresses with their own pitches (either may be a peer GPU's mapped memory); executed by a copy engine."""
    with torch.cuda.device(device):
        check(load().dw_mxfp8_copy_2d_async(dst_ptr, dst_pitch, src_ptr, src_pitch, width_bytes, height, _stream(device)),
              "dw_mxfp8_copy_2d_async")


QUANT_BATCH_MAX = 8


def quantize_rows_batch_into(xs, codes, scales, rule: int = RULE_OCP_FLOOR, layout: int = SF_TILED, flags: int = 0) -> int:
    """Row-wise quantisation of several matrices into caller-provided buffers with as few launches as possible
    (dw_mxfp8_quantize_rows_batch, up to QUANT_BATCH_MAX matrices per launch).  Every matrix must meet that entry point's
    conditions (cols % 32 == 0, 16-byte aligned; tiled scales: rows % 128 == 0 and cols % 128 == 0).  Returns the number
    of launches."""
    if not (len(xs) == len(codes) == len(scales)):
        raise RuntimeError("one codes and one scales buffer per input")
    if not xs:
        return 0
    dev = xs[0].device
    for x, c, s in zip(xs, codes, scales):
        _require_cuda(x, "input")
        if x.device != dev or c.device != dev or s.device != dev:
            raise RuntimeError("all tensors of a batch must be on one device")
        if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
            raise RuntimeError("inputs must be contiguous 2-D bfloat16 tensors")
        rows, cols = x.shape
        if c.numel() * c.element_size() != rows * cols or not c.is_contiguous() or not s.is_contiguous() \
                or s.numel() < scale_bytes(rows, cols, layout):
            raise RuntimeError("output buffers do not match the operand")
    L, launches = load(), 0
    with torch.cuda.device(dev):
        for at in range(0, len(xs), QUANT_BATCH_MAX):
            part = range(at, min(at + QUANT_BATCH_MAX, len(xs)))
            n = len(part)
            P, I = ctypes.c_void_p * n, ctypes.c_int64 * n
            check(L.dw_mxfp8_quantize_rows_batch(
                n, P(*[xs[i].data_ptr() for i in part]), P(*[codes[i].data_ptr() for i in part]),
                P(*[scales[i].data_ptr() for i in part]), I(*[xs[i].shape[0] for i in part]), I(*[xs[i].shape[1] for i in part]),
                rule, layout, flags, _stream(dev)), "dw_mxfp8_quantize_rows_batch")
            launches += 1
    return launches


def quantize_both(x: torch.Tensor, rule: int = RULE_OCP_FLOOR, layout: int = SF_TILED):
    """One read of x -> (codes_row, scales_row, codes_col_t, scales_col).  See dw_mxfp8_quantize_both."""
    return ext().quantize_both(x, rule, layout)


def quantize_both_colsum(x: torch.Tensor, rule: int = RULE_OCP_FLOOR, layout: int = SF_TILED, out_dtype=torch.float32):
    """quantize_both plus the column sums of x ([cols], fp32 or bf16) from the same read.  See dw_mxfp8_quantize_both_colsum."""
    return ext().quantize_both_colsum(x, rule, layout, out_dtype == torch.bfloat16)


def update_amax_history(x: torch.Tensor, amax_history: torch.Tensor) -> None:
    """amax_history (float32, on x's device) shifted by one, newest max |x| at [0].  See dw_mxfp8_update_amax_history."""
    _require_cuda(x, "input")
    _require_cuda(amax_history, "amax_history")
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise RuntimeError("input must be a contiguous bfloat16 tensor")
    if amax_history.dtype != torch.float32 or amax_history.dim() != 1 or not amax_history.is_contiguous():
        raise RuntimeError("amax_history must be a contiguous 1-D float32 tensor")
    with torch.cuda.device(x.device):
        check(load().dw_mxfp8_update_amax_history(x.data_ptr(), amax_history.data_ptr(), amax_history.numel(), x.numel(),
                                                  _stream(x.device)), "dw_mxfp8_update_amax_history")


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
    w = _status_words.get(device)
    if w is None:
        dev = torch.device(device)
        key = dev.index if dev.index is not None else torch.cuda.current_device()
        w = _status_words.get(key)
        if w is None:
            w = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
            _status_words[key] = w
        if dev.index is not None:
            _status_words[device] = w         # torch.device and "cuda:N" keys hit on the first lookup next time
    return w


def plan_word(variant: int = 0, group_m: int = 0, splits: int = 0, direct_stores: bool = False) -> int:
    """The plan word of dw_mxfp8_gemm_planned / dw_mxfp8_gemm_set_variant: kernel variant (0 = chosen per problem),
    row tiles per raster band, split-K count, per-thread instead of TMA stores."""
    return int(variant) | (int(group_m) << 8) | (int(splits) << 16) | (int(bool(direct_stores)) << 24)


def gemm(a_codes: torch.Tensor, a_sf: torch.Tensor, b_codes: torch.Tensor, b_sf: torch.Tensor,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, alpha: float = 1.0,
         beta: float = 0.0, plan: Optional[int] = None) -> torch.Tensor:
    """D[M,N] = alpha * A[M,K] . B[N,K]^T + beta * D + bias; operands as produced by quantize(..., SF_TILED).
    plan: this call's own plan word (plan_word(...)); None = the process default."""
    return ext().gemm(a_codes, a_sf, b_codes, b_sf, out, bias, float(alpha), float(beta), status_word(a_codes.device),
                      -1 if plan is None else int(plan))


def gemm_grouped(a_codes: torch.Tensor, a_sf: torch.Tensor, b_codes: torch.Tensor, b_sf: torch.Tensor,
                 tile_group: torch.Tensor, num_groups: int, rows_per_tile: int = 256, alpha: float = 1.0) -> torch.Tensor:
    """One launch over the groups: a_codes [M_total, K] (groups concatenated, each padded to rows_per_tile),
    b_codes [num_groups * N, K], tile_group int32 [M_total / rows_per_tile] on the device.  See dw_mxfp8_gemm_grouped."""
    for t, n in ((a_codes, "A"), (b_codes, "B"), (a_sf, "A scales"), (b_sf, "B scales"), (tile_group, "tile_group")):
        _require_cuda(t, n)
    M, K = a_codes.shape
    GN, Kb = b_codes.shape
    if K != Kb or GN % num_groups:
        raise RuntimeError(f"shape mismatch: A is [{M},{K}], stacked B is [{GN},{Kb}] for {num_groups} groups")
    N = GN // num_groups
    if tile_group.dtype != torch.int32 or tile_group.numel() != M // rows_per_tile or not tile_group.is_contiguous():
        raise RuntimeError("tile_group must be a contiguous int32 tensor with one entry per row tile")
    dev = a_codes.device
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        check(load().dw_mxfp8_gemm_grouped(a_codes.data_ptr(), a_sf.data_ptr(), b_codes.data_ptr(), b_sf.data_ptr(),
                                           out.data_ptr(), tile_group.data_ptr(), M, N, K, int(num_groups), int(rows_per_tile),
                                           float(alpha), status_word(dev).data_ptr(), _stream(dev)), "dw_mxfp8_gemm_grouped")
    return out


ACTIVATIONS = {"none": 0, "relu": 1, "gelu": 2, "silu": 3, "swiglu": 4}


def gemm_fused(a_codes: torch.Tensor, a_sf: torch.Tensor, b_codes: torch.Tensor, b_sf: torch.Tensor,
               bias: Optional[torch.Tensor] = None, activation: str = "none", quantize_out: bool = True,
               write_d: bool = True, alpha: float = 1.0, rule: int = RULE_OCP_FLOOR):
    """act(alpha * A . B^T + bias) -> (D bf16 or None, codes or None, tiled scales or None).  See dw_mxfp8_gemm_fused.
    activation="swiglu": B is the gate and up weight interleaved by interleave_gate_up(); the outputs have N / 2 columns."""
    for t, n in ((a_codes, "A"), (b_codes, "B"), (a_sf, "A scales"), (b_sf, "B scales")):
        _require_cuda(t, n)
    M, K = a_codes.shape
    N, Kb = b_codes.shape
    if K != Kb:
        raise RuntimeError(f"contraction mismatch: A is [{M},{K}], B is [{N},{Kb}]")
    if activation == "swiglu" and N % 64:
        raise RuntimeError("swiglu needs a fused gate+up width that is a multiple of 64")
    dev = a_codes.device
    n_out = N // 2 if activation == "swiglu" else N
    d = torch.empty((M, n_out), dtype=torch.bfloat16, device=dev) if write_d else None
    codes = torch.empty((M, n_out), dtype=torch.uint8, device=dev) if quantize_out else None
    scales = torch.empty(scale_bytes(M, n_out, SF_TILED), dtype=torch.uint8, device=dev) if quantize_out else None
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous()):
        raise RuntimeError("bias must be a contiguous bfloat16 [N] tensor")
    sw = status_word(dev)
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(dev):
        check(load().dw_mxfp8_gemm_fused(a_codes.data_ptr(), a_sf.data_ptr(), b_codes.data_ptr(), b_sf.data_ptr(), ptr(d),
                                         ptr(bias), M, N, K, float(alpha), 0.0, ACTIVATIONS[activation], ptr(codes),
                                         ptr(scales), rule, sw.data_ptr(), _stream(dev)), "dw_mxfp8_gemm_fused")
    return d, (None if codes is None else codes.view(torch.float8_e4m3fn)), scales


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[F, ...] gate and up weights (or [F] biases) -> the [2 F, ...] operand of the SwiGLU epilogue: groups of 32 gate
    rows followed by the 32 up rows of the same outputs (DW_ACT_SWIGLU of dw_mxfp8_gemm_fused).  F % 32 == 0."""
    if gate.shape != up.shape or gate.shape[0] % 32:
        raise RuntimeError("gate and up must have the same shape, with a multiple of 32 rows")
    f = gate.shape[0]
    rest = gate.shape[1:]
    return torch.stack((gate.reshape(f // 32, 32, *rest), up.reshape(f // 32, 32, *rest)), dim=1).reshape(2 * f, *rest)


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


def set_gemm_variant(v: int, group_m: int = 0, splits: int = 0, direct_stores: bool = False) -> None:
    """PROCESS default of the plan word, for calls that pass none (a switch for benchmarks and tests; library code
    passes `plan=` per call instead)."""
    check(load().dw_mxfp8_gemm_set_variant(plan_word(v, group_m, splits, direct_stores)), "dw_mxfp8_gemm_set_variant")
