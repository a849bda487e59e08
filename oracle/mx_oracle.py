"""CPU oracle for the MXFP8 linear path (quantise -> block-scaled GEMM).

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels; it is
imported by the test-suite, by the smoke check and by the CPU-baseline leg of the
benchmark, never by the product package.

It restates, in numpy integer/bit arithmetic, the algorithm of the reference path:

  * block geometry and amax           csrc/mxfp8_quantization.cu:37-38, :57-97
  * power-of-two block scale          csrc/mxfp8_quantization.cu:103-131
  * scaling + clamp to +-448          csrc/mxfp8_quantization.cu:137-161
  * row-major / column-major blocks   csrc/mxfp8_quantization.cu:64, :140
  * dequantise                        csrc/mxfp8_quantization.cu:179-202
  * logical scale shapes              csrc/mxfp8_quantization.cu:287-298
  * flat-tensor refactorisation       csrc/cutlass_kernels.cpp:358-375
  * GEMM = fp32-accumulated product   csrc/blackwell_gemm_kernel.cu:134-149,
    with alpha/beta, bf16 output      src/deepwell/cutlass_kernels.py:28-32

Two deliberate departures from the reference's literal code, both stated by the
target of this build (E4M3 payloads, E8M0 scales, scale = 2^(floor(log2 amax) - 8)):

  * payload is a real E4M3 code (round-to-nearest-even, saturating at +-448), not
    the reference's `static_cast<int8_t>` truncation (mxfp8_quantization.cu:159),
    which overflows for |q| > 127;
  * scale is stored as one E8M0 byte (biased exponent), not an fp32 value.

Two scale rules are provided.  "ocp_floor" is the contract rule; "ref_ceil" is the
reference's `2^ceil(log2(amax/448))` (mxfp8_quantization.cu:109-114) as the reference's
own kernel evaluates it (see e8m0_from_amax_bits): it equals ocp_floor except when the
7-bit bf16 mantissa of amax exceeds 0x60 (m > 1.75), where it is one exponent higher,
plus the two fast-math effects of the reference's build.

Parity pin: the reference's own tests hold no golden vector for this path, so the
reference itself was run.  (1) Its quantiser kernel, compiled from its source with its
own flags (oracle/Makefile -> oracle/_ref/), runs on the GPU in
tests/test_gpu_reference_quantizer.py; its output on every finite bf16 magnitude and on a
seeded matrix is recorded in tests/golden/ref_quantizer.npz
(tests/golden/make_reference_quantizer_golden.py) and tests/test_oracle.py holds this
module to it: ref_ceil scales bit for bit, scaled values against the reference's int8
payload.  (2) The reference's CPU GEMM module, run in the build container, is recorded in
tests/golden/ref_gemm.npz (tests/golden/make_golden.py).  (3) What the reference does not
have - a true E4M3 encoder, E8M0 bytes, the ocp_floor rule - is held against torch's
independent float8_e4m3fn / float8_e8m0fnu CPU casts and hand-derived vectors.
"""
from __future__ import annotations

import numpy as np

BLOCK = 32                      # mxfp8_quantization.cu:37
E4M3_MAX = 448.0                # mxfp8_quantization.cu:38
SCALE_RULES = ("ocp_floor", "ref_ceil")
RULE_ID = {"ocp_floor": 0, "ref_ceil": 1}


# ----------------------------------------------------------------------------
# bf16 <-> fp32 on bit patterns
# ----------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 patterns -> float32 values (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 patterns, round-to-nearest-even (NaN kept quiet)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    r = np.where(nan, ((u >> 16) | 0x0040).astype(np.uint16), r)
    return r


# ----------------------------------------------------------------------------
# E4M3 encode / decode
# ----------------------------------------------------------------------------
def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 (fn) code, RNE, saturating to +-448 (0x7E); NaN -> 0x7F.

    Same result as the hardware `cvt.rn.satfinite.e4m3x2.f32`, which writes the canonical
    NaN 0x7F whatever the sign of the NaN input (measured on B200; torch's CPU cast keeps
    the sign, the only place the two differ).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    sign = ((u >> 24) & 0x80).astype(np.uint8)
    au = u & 0x7FFFFFFF
    a = au.view(np.float32)
    nan = au > 0x7F800000
    # normal E4M3 range: |x| >= 2^-6.  Round the 23-bit mantissa to 3 bits, RNE.
    lsb = (au >> 20) & 1
    ru = (au + 0x7FFFF + lsb) & 0xFFF00000
    e = (ru >> 23).astype(np.int32) - 127
    m = (ru >> 20) & 7
    code_n = (((e + 7) << 3).astype(np.int64) | m.astype(np.int64))
    # subnormal E4M3: multiples of 2^-9, RNE (np.rint is ties-to-even)
    with np.errstate(invalid="ignore", over="ignore"):
        code_s = np.rint(a * np.float32(512.0)).astype(np.int64)
    small = au < np.float32(2.0 ** -6).view(np.uint32)
    code = np.where(small, code_s, code_n)
    sat = (~small) & (ru.view(np.float32) > np.float32(E4M3_MAX))
    code = np.where(sat, 0x7E, code)
    out = code.astype(np.uint8) | sign
    return np.where(nan, np.uint8(0x7F), out)


_E4M3_TABLE = None


def e4m3_decode_table() -> np.ndarray:
    """256-entry float32 table: E4M3 code -> value (0x7F/0xFF = NaN)."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        t = np.zeros(256, dtype=np.float32)
        for c in range(256):
            s = -1.0 if c & 0x80 else 1.0
            e = (c >> 3) & 0xF
            m = c & 7
            if e == 0xF and m == 7:
                v = np.nan
            elif e == 0:
                v = s * m * 2.0 ** -9
            else:
                v = s * (1 + m / 8.0) * 2.0 ** (e - 7)
            t[c] = v
        _E4M3_TABLE = t
    return _E4M3_TABLE


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return e4m3_decode_table()[codes.astype(np.uint8)]


# ----------------------------------------------------------------------------
# E8M0 scale bytes
# ----------------------------------------------------------------------------
def e8m0_from_amax_bits(amax_bits: np.ndarray, rule: str = "ocp_floor") -> np.ndarray:
    """bf16 pattern of a block's amax (sign cleared, NaNs excluded) -> E8M0 byte.

    byte = e + 127 with the scale 2^e, clamped to [0, 254].
      ocp_floor: e = floor(log2 amax) - 8
      ref_ceil : e = ceil(log2(amax / 448))        (mxfp8_quantization.cu:109-114), with the two places where
                 the reference's kernel, built with its own flags (--use_fast_math, setup.py:290) for sm_100a,
                 leaves that formula (measured by running that kernel on every bf16 magnitude,
                 tests/test_gpu_reference_quantizer.py): a quotient amax/448 below 2^-126 is flushed to zero and
                 the kernel then writes scale 1.0 (:111-116), i.e. amax pattern < 0x04E0 -> byte 127; and
                 amax = 1.75 * 2^k <= 224, whose quotient is exactly a power of two below 1, comes out one step
                 higher (the approximate division and logarithm land just above the integer).
    amax == 0 -> scale 1.0 -> byte 127             (mxfp8_quantization.cu:119-122)
    A bf16 subnormal amax has floor(log2) <= -127, so e + 127 < 0 -> byte 0 under ocp_floor.
    """
    if rule not in RULE_ID:
        raise ValueError(f"unknown scale rule {rule!r}")
    a = amax_bits.astype(np.int32) & 0x7FFF
    ef = a >> 7
    m7 = a & 0x7F
    byte = ef - 8
    if rule == "ref_ceil":
        up = (m7 > 0x60) | ((m7 == 0x60) & (ef <= 134))
        byte = byte + (up & (ef < 255)).astype(np.int32)
    byte = np.clip(byte, 0, 254)
    if rule == "ref_ceil":
        byte = np.where(a < 0x04E0, 127, byte)
    byte = np.where(a == 0, 127, byte)
    return byte.astype(np.uint8)


def e8m0_to_f32(byte: np.ndarray) -> np.ndarray:
    """E8M0 byte -> float32 2^(byte-127); byte 0 is the fp32 subnormal 2^-127."""
    b = byte.astype(np.uint32)
    bits = np.where(b == 0, np.uint32(0x00400000), b << 23).astype(np.uint32)
    return bits.view(np.float32)


def e8m0_inverse_f32(byte: np.ndarray) -> np.ndarray:
    """E8M0 byte -> float32 2^(127-byte) (exact; byte 254 gives the subnormal 2^-127)."""
    b = byte.astype(np.uint32)
    bits = np.where(b >= 254, np.uint32(0x00400000), (254 - b) << 23).astype(np.uint32)
    return bits.view(np.float32)


# ----------------------------------------------------------------------------
# quantise / dequantise
# ----------------------------------------------------------------------------
def _block_amax_bits(bits2d: np.ndarray) -> np.ndarray:
    """bits2d: [R, C] uint16 with C % 32 == 0 after padding -> [R, C/32] amax patterns.

    fmaxf(local_max, fabsf(v)) ignores NaN operands (mxfp8_quantization.cu:73), so NaN
    elements do not contribute.  For non-NaN bf16 the magnitude order equals the
    integer order of the 15 low bits.
    """
    a = (bits2d & 0x7FFF).astype(np.uint16)
    a = np.where(a > 0x7F80, 0, a)
    r, c = a.shape
    return a.reshape(r, c // BLOCK, BLOCK).max(axis=2)


def quantize_rowwise(bits: np.ndarray, rule: str = "ocp_floor"):
    """Row-wise MX quantisation: blocks of 32 along the last dim of a [R, C] matrix.

    bits: uint16 [R, C] bf16 patterns.  A ragged last block (C % 32 != 0) covers the
    remaining columns only (mxfp8_quantization.cu:53-55).
    Returns (codes uint8 [R, C], scales uint8 [R, ceil(C/32)]).
    """
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    r, c = bits.shape
    nb = (c + BLOCK - 1) // BLOCK
    if r == 0 or c == 0:
        return np.zeros((r, c), np.uint8), np.zeros((r, nb), np.uint8)
    pad = nb * BLOCK - c
    pb = np.pad(bits, ((0, 0), (0, pad))) if pad else bits
    scales = e8m0_from_amax_bits(_block_amax_bits(pb), rule)
    inv = e8m0_inverse_f32(scales)                       # [R, nb]
    x = bf16_bits_to_f32(pb).reshape(r, nb, BLOCK)
    with np.errstate(invalid="ignore", over="ignore"):
        q = x * inv[:, :, None]
    codes = e4m3_encode(q).reshape(r, nb * BLOCK)[:, :c]
    return np.ascontiguousarray(codes), scales


def quantize_colwise(bits: np.ndarray, rule: str = "ocp_floor", transpose_out: bool = True):
    """Column-wise MX quantisation of a row-major [R, C] matrix: blocks of 32 along dim 0.

    This is the reference's `row_major=false` addressing (idx = col*M + row,
    mxfp8_quantization.cu:64) seen from the memory side: the logical matrix is the
    transpose of what is stored, so blocks run down the stored rows.

    transpose_out=True  -> codes [C, R] (contraction dim contiguous), scales [C, ceil(R/32)]
                           — the operand form a K-major GEMM consumes (the body the
                           reference leaves empty at mxfp8_quantization.cu:216-226).
    transpose_out=False -> codes [R, C] in the input's own layout (what the reference's
                           kernel writes, :159), scales still [C, ceil(R/32)] (:125).
    """
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    codes_t, scales = quantize_rowwise(np.ascontiguousarray(bits.T), rule)
    if transpose_out:
        return codes_t, scales
    return np.ascontiguousarray(codes_t.T), scales


def dequantize_rowwise(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """codes uint8 [R, C], scales uint8 [R, ceil(C/32)] -> float32 [R, C] (exact products).

    out = value(code) * 2^e of block col/32 (mxfp8_quantization.cu:190-202).
    """
    r, c = codes.shape
    s = e8m0_to_f32(scales)
    s_full = np.repeat(s, BLOCK, axis=1)[:, :c]
    with np.errstate(invalid="ignore", over="ignore"):
        return e4m3_decode(codes) * s_full


def flat_factorisation(numel: int):
    """Rows x cols the reference gives a flat tensor (cutlass_kernels.cpp:358-375)."""
    if numel > 65536:
        m = 256
        while numel % m != 0 and m < 4096:
            m *= 2
        if numel % m == 0:
            return m, numel // m
    return 1, numel


# ----------------------------------------------------------------------------
# tcgen05 scale-factor layout (what the GEMM kernel reads)
# ----------------------------------------------------------------------------
def sf_tiled_size(rows: int, kblocks: int) -> int:
    """Bytes of the tiled scale buffer: 512-byte tiles of 128 rows x 4 k-blocks."""
    return ((rows + 127) // 128) * ((kblocks + 3) // 4) * 512


def sf_flat_to_tiled(scales: np.ndarray, pad_byte: int = 127) -> np.ndarray:
    """[R, KB] flat E8M0 bytes -> tiled byte buffer.

    Tile (R/128, KB/4) is 512 contiguous bytes; inside it row r, k-block c sits at
    (r%32)*16 + ((r/32)%4)*4 + (c%4).  Tiles are ordered row-tile major.  Padding rows
    and k-blocks hold `pad_byte` (a finite scale; the payload there is zero).
    """
    r, kb = scales.shape
    rt, kt = (r + 127) // 128, (kb + 3) // 4
    out = np.full(rt * kt * 512, pad_byte, dtype=np.uint8)
    rr, cc = np.meshgrid(np.arange(r), np.arange(kb), indexing="ij")
    off = ((rr // 128) * kt + cc // 4) * 512 + (rr % 32) * 16 + ((rr // 32) % 4) * 4 + (cc % 4)
    out[off.ravel()] = scales.ravel()
    return out


def sf_tiled_to_flat(buf: np.ndarray, rows: int, kblocks: int) -> np.ndarray:
    kt = (kblocks + 3) // 4
    rr, cc = np.meshgrid(np.arange(rows), np.arange(kblocks), indexing="ij")
    off = ((rr // 128) * kt + cc // 4) * 512 + (rr % 32) * 16 + ((rr // 32) % 4) * 4 + (cc % 4)
    return buf[off]


# ----------------------------------------------------------------------------
# GEMM
# ----------------------------------------------------------------------------
def gemm_dequantized(a_codes, a_scales, b_codes, b_scales, alpha: float = 1.0, beta: float = 0.0,
                     d_bits=None, bias_bits=None) -> np.ndarray:
    """D[M,N] = bf16( alpha * sum_k dq(A)[m,k] * dq(B)[n,k] + beta * D + bias ), both operands K-major.

    fp32 accumulation (csrc/blackwell_gemm_kernel.cu:134-149, CUBLAS_COMPUTE_32F); beta
    scales the previous content of D (csrc/cutlass_kernels.cpp:197; `c` is ignored there).
    Returns bf16 patterns (uint16) [M, N].
    """
    a = dequantize_rowwise(a_codes, a_scales)
    b = dequantize_rowwise(b_codes, b_scales)
    try:
        import torch
        acc = torch.matmul(torch.from_numpy(a), torch.from_numpy(b).t()).numpy()
    except ImportError:                                     # numpy-only fallback for the checker
        acc = a @ b.T
    acc = np.float32(alpha) * acc
    if beta != 0.0 and d_bits is not None:
        acc = acc + np.float32(beta) * bf16_bits_to_f32(d_bits)
    if bias_bits is not None:
        acc = acc + bf16_bits_to_f32(bias_bits)[None, :]
    return f32_to_bf16_bits(acc.astype(np.float32))


def mxfp8_linear(x_bits, w_bits, rule: str = "ocp_floor", bias_bits=None) -> np.ndarray:
    """Y[M,N] = X[M,K] . W[N,K]^T through MXFP8 operands (both row-wise along K)."""
    xc, xs = quantize_rowwise(x_bits, rule)
    wc, ws = quantize_rowwise(w_bits, rule)
    return gemm_dequantized(xc, xs, wc, ws, bias_bits=bias_bits)


# ----------------------------------------------------------------------------
# torch convenience (bf16 tensors in, numpy out) — used by tests and the smoke check
# ----------------------------------------------------------------------------
def torch_bf16_bits(t) -> np.ndarray:
    import torch
    assert t.dtype == torch.bfloat16
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_torch_bf16(bits: np.ndarray):
    import torch
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
