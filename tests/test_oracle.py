"""CPU tests: the oracle against the golden fixtures, torch's independent casts and its C twin."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import mx_oracle as o
from oracle import mx_ref as c
from conftest import config1_inputs


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("rule", o.SCALE_RULES)
def test_kat_rowwise_and_colwise(golden, rule):
    k = golden["kat_quant"]
    bits = k["bits"]
    codes, scales = o.quantize_rowwise(bits, rule)
    assert np.array_equal(codes, k[f"row_codes_{rule}"])
    assert np.array_equal(scales, k[f"row_scales_{rule}"])
    ccodes, cscales = o.quantize_colwise(bits, rule)
    assert np.array_equal(ccodes, k[f"col_codes_{rule}"])
    assert np.array_equal(cscales, k[f"col_scales_{rule}"])
    # the C restatement gives the same bytes
    cc, cs = c.quantize_rowwise(bits, o.RULE_ID[rule])
    assert np.array_equal(cc, codes) and np.array_equal(cs, scales)
    cc, cs = c.quantize_colwise(bits, o.RULE_ID[rule], True)
    assert np.array_equal(cc, ccodes) and np.array_equal(cs, cscales)


def test_known_answers_by_hand():
    f = np.zeros((1, 64), np.float32)
    f[0, :7] = [17, 19, 21, 23, 25, 27, 256]       # amax 256 = 2^8 -> e = 0, scale 1
    f[0, 32:38] = [448, 464, 480, 1000, -1000, 300]  # amax 1000 -> floor(log2)=9 -> e = 1, scale 2
    codes, scales = o.quantize_rowwise(o.f32_to_bf16_bits(f))
    assert scales.tolist() == [[127, 128]]
    # 17 -> 16 (tie to even), 19 -> 20, 21 -> 20, 23 -> 24, 25 -> 24, 27 -> 28, 256 -> 256
    assert o.e4m3_decode(codes[0, :7]).tolist() == [16, 20, 20, 24, 24, 28, 256]
    # /2: 224, 232->224|240 tie->224? 232 = 1.8125*128 -> between 224 and 240, nearer 240? |232-224|=8,|240-232|=8 tie -> even mantissa (224: m=6) ; 240, 500->448 sat, -448, 150->144|160: 150 nearer 144
    assert o.e4m3_decode(codes[0, 32:38]).tolist() == [224, 224, 240, 448, -448, 144]
    # reference rule never saturates: 1000/448 = 2.23 -> ceil(log2) = 2 -> scale 4
    codes_r, scales_r = o.quantize_rowwise(o.f32_to_bf16_bits(f), "ref_ceil")
    assert scales_r.tolist() == [[127 + 0, 127 + 2]]
    assert o.e4m3_decode(codes_r[0, 35:37]).tolist() == [256, -256]   # 250 -> tie 240|256 -> 256 (even)


def test_rules_differ_only_above_mantissa_1p75():
    """ref_ceil against ocp_floor: one step higher above mantissa 1.75 (the ceiling of the logarithm), and the two
    places where the reference's fast-math kernel leaves its own formula: amax = 1.75 * 2^k <= 224 also one step
    higher, amax below 448 * 2^-126 (pattern 0x04E0) scale 1."""
    amax = np.arange(1, 0x7F80, dtype=np.uint16)
    a = o.e8m0_from_amax_bits(amax, "ocp_floor").astype(int)
    b = o.e8m0_from_amax_bits(amax, "ref_ceil").astype(int)
    ef, m7 = amax >> 7, amax & 0x7F
    flushed = amax < 0x04E0
    high = ((m7 > 0x60) | ((m7 == 0x60) & (ef <= 134))) & ~flushed
    assert np.all(b[flushed] == 127)
    assert np.all((b - a)[high] == 1)
    assert np.all((b - a)[~high & ~flushed] == 0)
    assert o.e8m0_from_amax_bits(np.array([0], np.uint16)).tolist() == [127]


def test_e4m3_matches_torch_cast_on_every_bf16_value():
    bits = np.arange(65536, dtype=np.uint16)
    x = o.bf16_bits_to_f32(bits)
    mine = o.e4m3_encode(x)
    ref = torch.clamp(torch.from_numpy(x.copy()), -448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    nan = np.isnan(x)
    assert np.array_equal(mine[~nan], ref[~nan])
    assert np.all(mine[nan] == 0x7F)
    assert np.array_equal(o.e4m3_encode(o.e4m3_decode(np.arange(256, dtype=np.uint8)))[:0x7F], np.arange(0x7F, dtype=np.uint8))


def test_e8m0_matches_torch_dtype():
    b = np.arange(255, dtype=np.uint8)
    got = torch.from_numpy(o.e8m0_to_f32(b)).to(torch.float8_e8m0fnu).view(torch.uint8).numpy()
    assert np.array_equal(got, b)
    assert np.all(o.e8m0_to_f32(b) * o.e8m0_inverse_f32(b) == 1.0)


def test_config1_digests(golden):
    g = golden["config1"]
    X, W = config1_inputs()
    xb, wb = o.torch_bf16_bits(X), o.torch_bf16_bits(W)
    assert sha(xb) == str(g["x_bits_sha"]) and sha(wb) == str(g["w_bits_sha"]), "seeded inputs changed"
    xc, xs = c.quantize_rowwise(xb, 0)
    wc, ws = c.quantize_rowwise(wb, 0)
    assert sha(xc) == str(g["x_codes_sha"]) and sha(xs) == str(g["x_scales_sha"])
    assert sha(wc) == str(g["w_codes_sha"]) and sha(ws) == str(g["w_scales_sha"])
    # numpy oracle on a slice (the full matrix is covered by its C twin above)
    nc, ns = o.quantize_rowwise(xb[:128])
    assert np.array_equal(nc, xc[:128]) and np.array_equal(ns, xs[:128])
    y = o.gemm_dequantized(xc[:64], xs[:64], wc[:64], ws[:64])
    yf, gf = o.bf16_bits_to_f32(y), o.bf16_bits_to_f32(g["y_corner"])
    assert np.max(np.abs(yf - gf)) <= 1e-2 * np.max(np.abs(gf))


def test_gemm_oracle_matches_reference_cpu_module(golden):
    """ref_gemm.npz holds the output of the reference's own deepwell.cutlass_kernels.BlackwellGemmKernel.gemm
    (CPU) on the dequantised operands; the oracle must agree to bf16 rounding."""
    r = golden["ref_gemm"]
    ac, asc = o.quantize_rowwise(r["a_bits"])
    bc, bsc = o.quantize_rowwise(r["b_bits"])
    assert np.array_equal(ac, r["a_codes"]) and np.array_equal(bsc, r["b_scales"])
    y = o.bf16_bits_to_f32(o.gemm_dequantized(ac, asc, bc, bsc))
    ref = r["y_ref"]
    assert np.max(np.abs(y - ref)) <= 2.0 ** -8 * np.max(np.abs(ref))
    d0 = o.f32_to_bf16_bits(r["c"])
    y2 = o.bf16_bits_to_f32(o.gemm_dequantized(ac, asc, bc, bsc, alpha=0.5, beta=2.0, d_bits=d0))
    ref2 = 0.5 * ref + 2.0 * o.bf16_bits_to_f32(d0)
    assert np.max(np.abs(y2 - ref2)) <= 2.0 ** -7 * np.max(np.abs(ref2))
    # C twin
    y3 = o.bf16_bits_to_f32(c.gemm(ac, asc, bc, bsc))
    assert np.max(np.abs(y3 - ref)) <= 2.0 ** -8 * np.max(np.abs(ref))


@pytest.mark.parametrize("shape", [(0, 64), (5, 0), (1, 1), (3, 31), (7, 50), (33, 96), (130, 257)])
def test_ragged_and_empty(shape):
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 65536, shape, dtype=np.uint16)
    codes, scales = o.quantize_rowwise(bits)
    assert codes.shape == shape and scales.shape == (shape[0], (shape[1] + 31) // 32)
    if 0 not in shape:
        cc, cs = c.quantize_rowwise(bits, 0)
        assert np.array_equal(cc, codes) and np.array_equal(cs, scales)
        ct, st = o.quantize_colwise(bits)
        c2, s2 = c.quantize_colwise(bits, 0, True)
        assert np.array_equal(ct, c2) and np.array_equal(st, s2)
        cn, sn = o.quantize_colwise(bits, transpose_out=False)
        assert np.array_equal(cn, ct.T) and np.array_equal(sn, st)


def test_roundtrip_error_bound():
    """dq(q(x)) is within half an E4M3 ulp of x for unsaturated elements (ref_ceil never saturates)."""
    rng = np.random.default_rng(5)
    x = (rng.standard_t(3, (64, 512)) * 0.5).astype(np.float32)
    bits = o.f32_to_bf16_bits(x)
    xf = o.bf16_bits_to_f32(bits)
    codes, scales = o.quantize_rowwise(bits, "ref_ceil")
    dq = o.dequantize_rowwise(codes, scales)
    s = np.repeat(o.e8m0_to_f32(scales), 32, axis=1)
    assert np.all(np.abs(dq - xf) <= np.maximum(np.abs(xf) * 2.0 ** -4, s * 2.0 ** -10) + 1e-30)


def test_tiled_scale_layout_roundtrip_and_offsets():
    rng = np.random.default_rng(9)
    sc = rng.integers(0, 255, (300, 13), dtype=np.uint8)
    buf = o.sf_flat_to_tiled(sc)
    assert buf.size == o.sf_tiled_size(300, 13) == 3 * 4 * 512
    assert np.array_equal(o.sf_tiled_to_flat(buf, 300, 13), sc)
    # row 161, k-block 6: tile (1, 1) of a 4-wide tile grid; inside: (161%32)*16 + ((161/32)%4)*4 + 6%4
    assert buf[(1 * 4 + 1) * 512 + 1 * 16 + 1 * 4 + 2] == sc[161, 6]
    assert np.all(o.sf_flat_to_tiled(sc, pad_byte=7)[np.setdiff1d(np.arange(buf.size),
                  np.unique(((np.arange(300)[:, None] // 128) * 4 + np.arange(13)[None, :] // 4) * 512
                            + (np.arange(300)[:, None] % 32) * 16 + ((np.arange(300)[:, None] // 32) % 4) * 4
                            + np.arange(13)[None, :] % 4))] == 7)


def test_flat_factorisation_follows_reference():
    assert o.flat_factorisation(1000) == (1, 1000)
    assert o.flat_factorisation(65536) == (1, 65536)
    assert o.flat_factorisation(256 * 1000) == (256, 1000)
    assert o.flat_factorisation(256 * 1000 + 128) == (1, 256 * 1000 + 128)   # no power of two >= 256 divides
    assert o.flat_factorisation(65537 * 3) == (1, 65537 * 3)


def test_ref_ceil_rule_against_the_recorded_output_of_the_reference_kernel():
    """tests/golden/ref_quantizer.npz holds what the reference's own quantiser kernel wrote on a B200
    (tests/golden/make_reference_quantizer_golden.py): the oracle's ref_ceil scales must equal it on every finite
    bf16 magnitude and on the recorded matrix, row-wise and column-wise, and the oracle's scaled values must truncate
    to the recorded int8 payload wherever that fits in int8."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_quantizer.npz"))
    pats = np.arange(0x7F80, dtype=np.uint16)
    got = o.e8m0_from_amax_bits(pats, "ref_ceil").astype(np.int32) - 127
    assert np.array_equal(got, g["scale_log2_every_magnitude"].astype(np.int32))
    bits = g["x_bits"]
    codes, scales = o.quantize_rowwise(bits, "ref_ceil")
    assert np.array_equal(scales.astype(np.int32) - 127, g["scale_log2"].astype(np.int32))
    _, col_scales = o.quantize_colwise(bits, "ref_ceil")
    assert np.array_equal(col_scales.astype(np.int32) - 127, g["col_scale_log2"].astype(np.int32))
    x = o.bf16_bits_to_f32(bits).astype(np.float64).reshape(bits.shape[0], -1, 32)
    scaled = x / np.exp2(g["scale_log2"].astype(np.float64))[:, :, None]
    fits = np.abs(scaled) < 127
    assert np.array_equal(np.trunc(scaled)[fits].astype(np.int8), g["payload"].reshape(scaled.shape)[fits])
    # the C restatement follows the same rule
    from oracle import mx_ref
    ccodes, cscales = mx_ref.quantize_rowwise(bits, 1)
    assert np.array_equal(cscales, scales) and np.array_equal(ccodes, codes)
