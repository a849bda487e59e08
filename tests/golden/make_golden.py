"""Generates the golden fixtures of tests/golden/ (run in the build container, where the
reference checkout is readable):

    python tests/golden/make_golden.py /path/to/reference

kat_quant.npz      known-answer matrix for the quantiser (ties, saturation, zero / subnormal /
                   NaN / Inf blocks, amax mantissas on both sides of 1.75, every exponent).
                   Expected codes and scales are written only after two independent
                   computations agree: the oracle's bit arithmetic and float64 log2 + torch's
                   float8_e4m3fn / float8_e8m0fnu CPU casts.
config1.npz        BASELINE config 1 (X [2048,4096] N(0,1) with 1% x50 outliers, W [4096,4096]
                   N(0,0.02), seed 1234): SHA-256 of the full codes / scales, a 64x64 corner of Y.
ref_gemm.npz       output of the reference's own CPU GEMM module
                   (src/deepwell/cutlass_kernels.py:28-32) on dequantised MXFP8 operands.
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))
from oracle import mx_oracle as o  # noqa: E402


def independent_quantize_rowwise(bits, rule):
    """float64 / torch-cast computation, sharing no code with the oracle."""
    x = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(torch.float64)
    r, c = x.shape
    xb = x.reshape(r, c // 32, 32)
    a = xb.abs()
    a = torch.where(torch.isnan(a), torch.zeros_like(a), a)
    amax = a.amax(dim=2)
    with np.errstate(divide="ignore"):
        l2 = torch.log2(amax)
    if rule == "ocp_floor":
        e = torch.floor(l2) - 8
    else:
        # the formula, plus the two places where the reference's fast-math kernel leaves it on sm_100a
        # (oracle/mx_oracle.py::e8m0_from_amax_bits): quotient below 2^-126 -> scale 1; quotient an exact power
        # of two below 1 -> one step higher
        quot = amax / 448.0
        lq = torch.log2(quot)
        e = torch.ceil(lq)
        e = torch.where((lq == torch.round(lq)) & (quot < 1.0), e + 1, e)
        e = torch.where(quot < 2.0 ** -126, torch.zeros_like(e), e)
    e = torch.where(torch.isinf(amax), torch.full_like(e, 120.0), e)
    byte = torch.clamp(e + 127, 0, 254)
    byte = torch.where(amax == 0, torch.full_like(byte, 127.0), byte).to(torch.uint8)
    scale = torch.pow(torch.tensor(2.0, dtype=torch.float64), byte.to(torch.float64) - 127)
    q = (xb / scale[:, :, None]).to(torch.float32)
    q = torch.where(torch.isnan(q), q, torch.clamp(q, -448, 448))
    codes = q.to(torch.float8_e4m3fn).view(torch.uint8).reshape(r, c).numpy()
    return codes, byte.numpy()


def kat_matrix():
    rows = []
    def blk(vals):
        v = np.zeros(32, np.float32); v[: len(vals)] = vals; return v
    f = [blk([17, 19, 21, 23, 25, 27, 256]),                      # RNE ties at 3 mantissa bits
         blk([448, 464, 480, 1000, -1000, 300]),                  # saturation under ocp_floor
         blk([]),                                                  # zero block -> scale byte 127
         blk([1.75, 0.1]), blk([1.7578125, 0.1]), blk([1.9921875, -0.3]), blk([1.0, 0.999]),
         blk([2.0 ** -130, 2.0 ** -133]), blk([2.0 ** -126, 2.0 ** -127]),   # subnormal amax
         blk([2.0 ** 127, 1.0]), blk([3.0e38, -3.0e38]),
         blk([np.inf, 1.0, -2.0]), blk([np.nan, 3.0, -5.0]), blk([-np.nan, np.inf]),
         blk([2.0 ** -9 * 448 / 512, 1.0]), blk([-0.0, 0.0, 1e-20])]
    for e in range(-126, 128, 6):
        f.append(blk([2.0 ** e, 1.5 * 2.0 ** e, -1.875 * 2.0 ** (e - 1), 2.0 ** (e - 9), 2.0 ** (e - 10) * 1.5]))
    rng = np.random.default_rng(7)
    while len(f) % 8:
        f.append((rng.standard_normal(32) * np.exp(rng.uniform(-8, 8))).astype(np.float32))
    m = np.stack(f).reshape(-1, 8 * 32)                            # [R, 256]
    pad = (-m.shape[0]) % 32
    if pad:
        m = np.concatenate([m, (rng.standard_normal((pad, 256)) * 3).astype(np.float32)])
    return o.f32_to_bf16_bits(m)


def main():
    if len(sys.argv) < 2 or not os.path.isdir(os.path.join(sys.argv[1], "src", "deepwell")):
        raise SystemExit("usage: make_golden.py <root of the reference checkout>")
    ref_root = sys.argv[1]
    # ---- KAT ----
    bits = kat_matrix()
    out = {"bits": bits}
    for rule in o.SCALE_RULES:
        codes, scales = o.quantize_rowwise(bits, rule)
        icodes, iscales = independent_quantize_rowwise(bits, rule)
        nan = (codes & 0x7F) == 0x7F
        assert np.array_equal(scales, iscales), f"scale disagreement under {rule}"
        assert np.array_equal(codes[~nan], icodes[~nan]) and np.all((icodes[nan] & 0x7F) == 0x7F), rule
        ccodes, cscales = o.quantize_colwise(bits, rule)
        out[f"row_codes_{rule}"], out[f"row_scales_{rule}"] = codes, scales
        out[f"col_codes_{rule}"], out[f"col_scales_{rule}"] = ccodes, cscales
    np.savez_compressed(os.path.join(HERE, "kat_quant.npz"), **out)

    # ---- BASELINE config 1 ----
    g = torch.Generator("cpu").manual_seed(1234)
    X = torch.randn(2048, 4096, generator=g)
    mask = torch.rand(2048, 4096, generator=g) < 0.01
    X[mask] *= 50
    W = torch.randn(4096, 4096, generator=g) * 0.02
    xb, wb = o.torch_bf16_bits(X.bfloat16()), o.torch_bf16_bits(W.bfloat16())
    xc, xs = o.quantize_rowwise(xb)
    wc, ws = o.quantize_rowwise(wb)
    ixc, ixs = independent_quantize_rowwise(xb, "ocp_floor")
    assert np.array_equal(xc, ixc) and np.array_equal(xs, ixs)
    y = o.gemm_dequantized(xc[:64], xs[:64], wc[:64], ws[:64])
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    np.savez_compressed(os.path.join(HERE, "config1.npz"), x_codes_sha=sha(xc), x_scales_sha=sha(xs), w_codes_sha=sha(wc),
                        w_scales_sha=sha(ws), x_bits_sha=sha(xb), w_bits_sha=sha(wb), y_corner=y,
                        x_scales_head=xs[:8], x_codes_head=xc[:8, :64])

    # ---- the reference's CPU GEMM on dequantised operands ----
    sys.path.insert(0, os.path.join(ref_root, "src"))
    sys.dont_write_bytecode = True
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_cutlass_kernels", os.path.join(ref_root, "src", "deepwell", "cutlass_kernels.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = torch.Generator("cpu").manual_seed(99)
    A = (torch.randn(96, 256, generator=g) * 2).bfloat16()
    B = (torch.randn(80, 256, generator=g) * 0.05).bfloat16()
    ac, asc = o.quantize_rowwise(o.torch_bf16_bits(A))
    bc, bsc = o.quantize_rowwise(o.torch_bf16_bits(B))
    a_dq = torch.from_numpy(o.dequantize_rowwise(ac, asc))
    b_dq = torch.from_numpy(o.dequantize_rowwise(bc, bsc))
    k = ref.BlackwellGemmKernel()
    k.initialize(96, 80, 256, "mxfp8", True, 32)
    C = torch.randn(96, 80, generator=g)
    y_ref = k.gemm(a_dq, b_dq.t(), None, 1.0, 0.0).numpy()
    y_ref_ab = k.gemm(a_dq, b_dq.t(), C, 0.5, 2.0).numpy()
    np.savez_compressed(os.path.join(HERE, "ref_gemm.npz"), a_bits=o.torch_bf16_bits(A), b_bits=o.torch_bf16_bits(B),
                        a_codes=ac, a_scales=asc, b_codes=bc, b_scales=bsc, c=C.numpy(), y_ref=y_ref, y_ref_ab=y_ref_ab)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
