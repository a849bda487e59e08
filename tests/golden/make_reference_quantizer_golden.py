"""Records what the reference's own quantiser kernel produces on a B200 (needs a GPU and oracle/_ref/, which
oracle/Makefile builds from the reference's csrc/mxfp8_quantization.cu with the reference's nvcc flags):

    python tests/golden/make_reference_quantizer_golden.py [output directory]

ref_quantizer.npz
    scale_log2_every_magnitude   int16 [32640]: log2 of the fp32 scale the kernel writes for a block whose amax is
                                 the bf16 magnitude pattern p (p = 0 .. 0x7F7F, every finite bf16 magnitude)
    x_bits, scale_log2, payload  a seeded [128, 256] bf16 matrix (N(0,1), 1 % of the entries x 50), the log2 of
                                 the kernel's row-wise scales [128, 8] and its int8 payload [128, 256]
    col_scale_log2               the same matrix through the kernel's row_major = false addressing: [256, 4]

The fixture lets the CPU tests hold the oracle's "ref_ceil" rule against the reference's real output without a GPU.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))
from oracle import mx_ref  # noqa: E402


def run_reference(L, x, row_major=True):
    """x: bf16 CUDA tensor [R, C].  row_major: blocks along C, scales [R, C/32]; else the kernel's column-major
    addressing: blocks along R, scales [C, R/32] (csrc/mxfp8_quantization.cu:64)."""
    M, N = (x.shape[0], x.shape[1]) if row_major else (x.shape[1], x.shape[0])
    out = torch.empty(x.shape, dtype=torch.int8, device="cuda")
    scales = torch.empty(M, (N + 31) // 32, dtype=torch.float32, device="cuda")
    rc = L.ref_quantize_to_mxfp8_bf16(out.data_ptr(), scales.data_ptr(), x.data_ptr(), M, N, int(row_major),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"CUDA error {rc}"
    torch.cuda.synchronize()
    return out, scales


def every_magnitude_matrix():
    """[1020, 1024] bf16: block k (32 elements) holds magnitude pattern k in its first element, zeros elsewhere."""
    pat = torch.arange(0x7F80, dtype=torch.int32)
    x = torch.zeros(0x7F80, 32, dtype=torch.int16)
    x[:, 0] = pat.to(torch.int16)
    return x.view(-1, 1024).view(torch.bfloat16)


def log2_int16(scales):
    s = scales.double().cpu()
    out = torch.where(torch.isinf(s), torch.full_like(s, 32767.0), torch.log2(s))
    assert torch.equal(out, torch.round(out)), "a scale that is not a power of two"
    return out.to(torch.int16).numpy()


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    L = mx_ref.reference_quantizer()
    if L is None:
        raise SystemExit("oracle/_ref/libref_mxfp8_quant.so is not built (make -C oracle reference REFERENCE=<checkout>)")
    _, sc = run_reference(L, every_magnitude_matrix().cuda())
    g = torch.Generator("cpu").manual_seed(2468)
    x = torch.randn(128, 256, generator=g)
    x[torch.rand(128, 256, generator=g) < 0.01] *= 50
    x = x.bfloat16()
    payload, scales = run_reference(L, x.cuda())
    _, col_scales = run_reference(L, x.cuda(), row_major=False)
    np.savez_compressed(os.path.join(out_dir, "ref_quantizer.npz"),
                        scale_log2_every_magnitude=log2_int16(sc).reshape(-1),
                        x_bits=x.view(torch.int16).numpy().view(np.uint16), scale_log2=log2_int16(scales),
                        payload=payload.cpu().numpy(), col_scale_log2=log2_int16(col_scales))
    print("wrote", os.path.join(out_dir, "ref_quantizer.npz"))


if __name__ == "__main__":
    main()
