"""GPU test of dw_mxfp8_gemm_splitk_static, the split-K GEMM for callers that cannot allocate.

An operator that runs inside a serving engine whose pool already owns all free device memory, or
a binding that has no allocator to ask, cannot give dw_mxfp8_gemm the workspace it wants when it
splits K.  This entry point keeps the partial sums in a fixed array inside the library instead.
The test calls it straight through the C ABI (ctypes, raw pointers), twice in a row on different
problems so that the second call finds the first call's leftovers in the shared array, and compares
each result with dw_mxfp8_gemm run with a caller-provided workspace and the same split count (the same
kernel and the same order of additions, so the outputs must be identical bit for bit) and with the CPU
oracle (within the GEMM tolerance).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
RTOL = 1e-2          # the tolerance of tests/test_gpu_gemm.py


def _operands(nv, M, N, K, seed):
    g = torch.Generator("cpu").manual_seed(seed)
    a = torch.randn(M, K, generator=g).bfloat16().cuda()
    b = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    ac, asf = nv.quantize(a, nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
    bc, bsf = nv.quantize(b, nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    d0 = torch.randn(M, N, generator=g).bfloat16().cuda()
    return ac, asf, bc, bsf, bias, d0


def _oracle(ops, alpha, beta):
    """alpha * dq(A) . dq(B)^T + beta * D0 + bias in fp32 on the CPU (the oracle's dequantiser on the operands' bytes)."""
    import numpy as np
    from oracle import mx_oracle as o
    ac, asf, bc, bsf, bias, d0 = ops
    host = lambda t: t.view(torch.uint8).cpu().numpy()
    M, K = ac.shape
    N = bc.shape[0]
    a = torch.from_numpy(o.dequantize_rowwise(host(ac), o.sf_tiled_to_flat(host(asf), M, K // 32)))
    b = torch.from_numpy(o.dequantize_rowwise(host(bc), o.sf_tiled_to_flat(host(bsf), N, K // 32)))
    return (alpha * (a @ b.t()) + beta * d0.float().cpu() + bias.float().cpu()[None, :]).double()


def _close(got, ref):
    got, ref = got.double(), ref.double()
    return bool(((got - ref).abs() <= RTOL * torch.maximum(ref.abs(), ref.abs().mean())).all())


def test_static_scratch_entry_point_matches_workspace_entry_point(native_lib):
    from deepwell_b200 import _native as nv
    assert torch.cuda.is_available() and native_lib.dw_mxfp8_device_supported(0) == 1
    L = native_lib
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    status = nv.status_word("cuda:0")
    nv.set_gemm_variant(0)

    def run_static(ops, M, N, K, splits, alpha, beta):
        ac, asf, bc, bsf, bias, d0 = ops
        out = d0.clone()
        rc = L.dw_mxfp8_gemm_splitk_static(ac.data_ptr(), asf.data_ptr(), bc.data_ptr(), bsf.data_ptr(), out.data_ptr(),
                                           bias.data_ptr(), M, N, K, alpha, beta, splits, status.data_ptr(), stream)
        assert rc == 0, L.dw_mxfp8_error_string(rc)
        return out

    def run_workspace(ops, M, N, K, splits, alpha, beta):
        ac, asf, bc, bsf, bias, d0 = ops
        out = d0.clone()
        nv.set_gemm_variant(0, splits=splits)
        try:
            ws_bytes = int(L.dw_mxfp8_gemm_workspace(M, N, K))
            assert ws_bytes > 0
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
            rc = L.dw_mxfp8_gemm(ac.data_ptr(), asf.data_ptr(), bc.data_ptr(), bsf.data_ptr(), out.data_ptr(),
                                 bias.data_ptr(), M, N, K, alpha, beta, ws.data_ptr(), ws_bytes, status.data_ptr(), stream)
            assert rc == 0, L.dw_mxfp8_error_string(rc)
        finally:
            nv.set_gemm_variant(0)
        return out

    # two calls in a row: the second, smaller problem reuses the array with the first one's contents in it
    cases = [(1024, 768, 8192, 4, 0.5, 2.0, 11), (384, 520, 4096, 3, 1.0, 0.0, 12)]
    for M, N, K, splits, alpha, beta, seed in cases:
        ops = _operands(nv, M, N, K, seed)
        got = run_static(ops, M, N, K, splits, alpha, beta)
        ref = run_workspace(ops, M, N, K, splits, alpha, beta)
        nv.check_status("cuda:0")
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), (M, N, K)
        assert _close(got.cpu(), _oracle(ops, alpha, beta)), (M, N, K)

    # sizes beyond the fixed array are refused, nothing is launched
    big_m, big_n = 4096, 4096                       # 2 splits x 64 MiB of partial sums > 32 MiB
    p16 = ctypes.c_void_p(16)
    rc = L.dw_mxfp8_gemm_splitk_static(p16, p16, p16, p16, p16, None, big_m, big_n, 4096, 1.0, 0.0, 2, None, stream)
    assert rc == -5
    assert L.dw_mxfp8_gemm_splitk_static(p16, p16, p16, p16, p16, None, 128, 128, 4096, 1.0, 0.0, 1, None, stream) == -1
