"""The reference's OWN quantiser kernel, run on the same GPU and the same inputs as this package's kernels.

oracle/Makefile compiles the reference's csrc/mxfp8_quantization.cu (where it lies, with the reference's nvcc flags)
plus a forwarding shim into oracle/_ref/libref_mxfp8_quant.so; the built file travels with the repository to the GPU
machine.  The reference writes fp32 power-of-two scales and an int8 payload (static_cast of the clamped quotient,
csrc/mxfp8_quantization.cu:152-159); this package writes E8M0 bytes and real E4M3 codes.  What must agree, bit for bit:

  * the scale of every block under DW_RULE_REF_CEIL: 2^(byte - 127) == the reference's fp32 scale, for every finite
    bf16 magnitude as amax, for random data, row-wise and column-wise;
  * the scaled value: trunc(x / scale) == the reference's int8 payload wherever it fits in int8 (the reference's cast
    of larger values is undefined in C++; under its rule the amax of every block is such a value).
"""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as o
from oracle import mx_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    L = mx_ref.reference_quantizer()
    if L is None:
        pytest.skip("oracle/_ref/libref_mxfp8_quant.so is not built")
    return L


@pytest.fixture(scope="module")
def nv(native_lib):
    from deepwell_b200 import _native
    return _native


def run_reference(L, x, row_major=True):
    M, N = (x.shape[0], x.shape[1]) if row_major else (x.shape[1], x.shape[0])
    out = torch.empty(x.shape, dtype=torch.int8, device="cuda")
    scales = torch.empty(M, (N + 31) // 32, dtype=torch.float32, device="cuda")
    rc = L.ref_quantize_to_mxfp8_bf16(out.data_ptr(), scales.data_ptr(), x.data_ptr(), M, N, int(row_major),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"CUDA error {rc}"
    torch.cuda.synchronize()
    return out, scales


def scale_of(byte):
    return torch.ldexp(torch.ones_like(byte, dtype=torch.float32), byte.int() - 127)


def test_scale_of_every_finite_magnitude_matches_the_reference_kernel(ref, nv):
    pat = torch.arange(0x7F80, dtype=torch.int32)
    x = torch.zeros(0x7F80, 32, dtype=torch.int16)
    x[:, 0] = pat.to(torch.int16)
    x = x.view(-1, 1024).view(torch.bfloat16).cuda()
    _, ref_scales = run_reference(ref, x)
    _, byte = nv.quantize(x, nv.DIR_ROW, nv.RULE_REF_CEIL, nv.SF_FLAT)
    assert torch.equal(scale_of(byte), ref_scales)
    # and the oracle's rule on the same patterns
    ob = o.e8m0_from_amax_bits(pat.numpy().astype(np.uint16), "ref_ceil")
    assert np.array_equal(ob, byte.cpu().numpy().reshape(-1))
    # a negative amax and an amax that is not the first element give the same scales
    x2 = torch.zeros(0x7F80, 32, dtype=torch.int16)
    x2[:, 17] = (pat | 0x8000).to(torch.int16)
    x2[:, 3] = (pat // 2).to(torch.int16)
    _, ref2 = run_reference(ref, x2.view(-1, 1024).view(torch.bfloat16).cuda())
    assert torch.equal(ref2, ref_scales)


@pytest.mark.parametrize("shape", [(2048, 4096), (512, 768), (96, 160)])
def test_random_data_scales_and_scaled_values_match_the_reference_kernel(ref, nv, shape):
    g = torch.Generator("cuda").manual_seed(shape[0] + shape[1])
    x = torch.randn(*shape, device="cuda", generator=g)
    x[torch.rand(*shape, device="cuda", generator=g) < 0.01] *= 50
    x = x.bfloat16()
    payload, ref_scales = run_reference(ref, x)
    codes, byte = nv.quantize(x, nv.DIR_ROW, nv.RULE_REF_CEIL, nv.SF_FLAT)
    assert torch.equal(scale_of(byte), ref_scales)
    scaled = x.float().view(shape[0], -1, 32) / ref_scales.unsqueeze(-1)
    fits = scaled.abs() < 127
    assert torch.equal(torch.trunc(scaled).to(torch.int8)[fits], payload.view(shape[0], -1, 32)[fits])
    # this package's E4M3 codes decode to the same scaled values after rounding to E4M3 (RNE, 3 mantissa bits):
    # |decode(code) - scaled| <= half an E4M3 step of the scaled value
    dec = torch.from_numpy(o.e4m3_decode(codes.view(torch.uint8).cpu().numpy())).view(shape[0], -1, 32)
    s = scaled.cpu()
    step = torch.maximum(torch.exp2(torch.floor(torch.log2(s.abs().clamp_min(2.0 ** -6))) - 3), torch.tensor(2.0 ** -9))
    assert bool(((dec - s.clamp(-448, 448)).abs() <= step / 2).all())
    # column-wise: the kernel's row_major = false addressing scales along dim 0 of the same row-major matrix
    if shape[0] % 32 == 0:
        _, ref_col = run_reference(ref, x, row_major=False)
        _, byte_col = nv.quantize(x, nv.DIR_COL, nv.RULE_REF_CEIL, nv.SF_FLAT)
        assert torch.equal(scale_of(byte_col), ref_col)
