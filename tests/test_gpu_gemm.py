"""GPU parity tests of the block-scaled GEMM (through the C ABI) against the oracle's
fp32-accumulated dequantised matmul.

Tolerance (bf16 output, accumulation order differs from the CPU's): |got - ref| <= 1e-2 * max(|ref|, mean|ref|)."""
import numpy as np
import pytest
import torch

from conftest import config1_inputs
from oracle import mx_oracle as o

pytestmark = pytest.mark.gpu
RTOL = 1e-2
VARIANTS = [1, 2, 3, 4, 5]   # 1 CTA x BN128, 1 CTA x BN256, CTA pair x BN256, CTA pair x BN128, CTA pair x BN192


@pytest.fixture(scope="module")
def nv(native_lib):
    from deepwell_b200 import _native
    assert torch.cuda.is_available() and native_lib.dw_mxfp8_device_supported(0) == 1
    yield _native
    _native.set_gemm_variant(0)


def host(t):
    return t.view(torch.uint8).cpu().numpy()


def assert_close(got, ref):
    got, ref = got.double(), ref.double()
    floor = ref.abs().mean()
    bad = (got - ref).abs() > RTOL * torch.maximum(ref.abs(), floor)
    assert not torch.isnan(got).any()
    assert bad.sum().item() == 0, f"{bad.sum().item()} of {bad.numel()} outside tolerance; max err {(got-ref).abs().max().item()}"


def oracle_gemm(nv, x, w, alpha=1.0, beta=0.0, d0=None, bias=None, rows=None, cols=None):
    """fp32-accumulated product of the dequantised operands (optionally a row/column sample).

    The codes and scales that are dequantised here come from the GPU quantiser.  That is sound because the
    quantiser is pinned bit for bit against the oracle on its own (tests/test_gpu_quantize.py), so these are the
    bytes the oracle's quantiser would give; test_smoke_matrix_end_to_end_through_the_oracle below keeps one case
    that goes bf16 -> oracle quantiser -> oracle GEMM with nothing from the GPU on the reference side."""
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_FLAT)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_FLAT)
    xc, xs, wc, ws = host(xc), host(xs), host(wc), host(ws)
    if rows is not None:
        xc, xs = xc[rows], xs[rows]
    if cols is not None:
        wc, ws = wc[cols], ws[cols]
    a = torch.from_numpy(o.dequantize_rowwise(xc, xs))
    b = torch.from_numpy(o.dequantize_rowwise(wc, ws))
    y = alpha * (a @ b.t())
    if beta != 0.0:
        y = y + beta * d0.float().cpu()
    if bias is not None:
        y = y + bias.float().cpu()[None, :]
    return y


def run(nv, M, N, K, alpha=1.0, beta=0.0, use_bias=False, seed=0):
    g = torch.Generator("cpu").manual_seed(seed + M * 31 + N * 17 + K)
    x = torch.randn(M, K, generator=g)
    x[torch.rand(M, K, generator=g) < 0.01] *= 50
    x = x.bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16().cuda()
    d0 = torch.randn(M, N, generator=g).bfloat16().cuda() if beta != 0.0 else None
    bias = torch.randn(N, generator=g).bfloat16().cuda() if use_bias else None
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    out = nv.gemm(xc, xs, wc, ws, out=None if d0 is None else d0.clone(), bias=bias, alpha=alpha, beta=beta)
    nv.check_status()
    assert_close(out.cpu(), oracle_gemm(nv, x, w, alpha, beta, d0, bias))


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 256, 256), (128, 256, 32), (512, 768, 1024), (300, 200, 160),
                                   (1000, 520, 96), (1, 32, 32), (129, 257 * 8, 4096 + 32), (2048, 512, 2048)])
def test_shapes(nv, variant, shape):
    nv.set_gemm_variant(variant)
    run(nv, *shape)


@pytest.mark.parametrize("variant", VARIANTS)
def test_alpha_beta_bias(nv, variant):
    nv.set_gemm_variant(variant)
    run(nv, 384, 640, 512, alpha=0.5, beta=2.0, use_bias=True)
    run(nv, 200, 104, 64, alpha=-1.25, beta=0.0, use_bias=True)       # N % 8 == 0 but ragged tiles
    run(nv, 96, 100, 64, alpha=1.0, beta=1.0, use_bias=False)          # N % 8 != 0: scalar store path


@pytest.mark.parametrize("variant", VARIANTS)
def test_tma_store_and_direct_store_epilogues_agree(nv, variant):
    """The bf16 output written through shared memory + TMA stores equals the per-thread-store path bit for bit,
    also where the last row/column tiles are ragged (the TMA store clips them)."""
    for M, N, K in [(512, 768, 256), (300, 200, 160), (129, 2056, 128), (1000, 520, 96)]:
        g = torch.Generator("cpu").manual_seed(M + N + K)
        x = torch.randn(M, K, generator=g).bfloat16().cuda()
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16().cuda()
        bias = torch.randn(N, generator=g).bfloat16().cuda()
        xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
        wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
        outs = []
        for direct in (False, True):
            nv.set_gemm_variant(variant, direct_stores=direct)
            guard = torch.full((M + 1, N), -7.0, dtype=torch.bfloat16, device="cuda")      # one row past the output
            nv.gemm(xc, xs, wc, ws, out=guard[:M], bias=bias)
            nv.check_status()
            assert (guard[M] == -7.0).all()
            outs.append(guard[:M].clone())
        nv.set_gemm_variant(0)
        assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16)), (M, N, K)


def test_smoke_matrix_end_to_end_through_the_oracle(nv):
    """X [2048,4096] N(0,1) with 1 % outliers x50, W [4096,4096] N(0,0.02): the reference side is computed entirely on
    the CPU (oracle quantiser on the bf16 bits, oracle dequantised fp32 GEMM) on a band of rows and columns that
    crosses tile edges; the GPU side is quantise + GEMM through the C ABI."""
    nv.set_gemm_variant(0)
    X, W = config1_inputs()
    rows = np.r_[0:40, 120:136, 250:262, 2040:2048]
    cols = np.r_[0:24, 248:264, 1016:1032, 4088:4096]
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    xq, xs = o.quantize_rowwise(bits(X[rows]))
    wq, ws = o.quantize_rowwise(bits(W[cols]))
    ref = torch.from_numpy(o.dequantize_rowwise(xq, xs)) @ torch.from_numpy(o.dequantize_rowwise(wq, ws)).t()
    x, w = X.cuda(), W.cuda()
    xc, xsf = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, wsf = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    y = nv.gemm(xc, xsf, wc, wsf)
    nv.check_status()
    assert_close(y.cpu()[rows][:, cols], ref)


@pytest.mark.parametrize("variant", [0, 3])
def test_config1_full(nv, golden, variant):
    """The 2048 x 4096 x 4096 outlier matrix in full: X [2048,4096] . W [4096,4096]^T, and the golden 64x64 corner."""
    nv.set_gemm_variant(variant)
    X, W = config1_inputs()
    x, w = X.cuda(), W.cuda()
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    y = nv.gemm(xc, xs, wc, ws)
    nv.check_status()
    assert_close(y.cpu(), oracle_gemm(nv, x, w))
    corner = torch.from_numpy(o.bf16_bits_to_f32(golden["config1"]["y_corner"]))
    assert_close(y[:64, :64].cpu(), corner)


def band_edge_samples(extent, tile_sizes, extra, gen):
    """Indices that include the first and the last element of every tile of every size in `tile_sizes` along an axis
    of length `extent` (so every tile band edge of the kernels' 128/192/256-wide tiles is hit), plus `extra` random ones."""
    idx = {0, extent - 1}
    for t in tile_sizes:
        for start in range(0, extent, t):
            idx.add(start)
            idx.add(min(start + t, extent) - 1)
    idx.update(int(v) for v in torch.randint(0, extent, (extra,), generator=gen))
    return torch.tensor(sorted(idx))


@pytest.mark.parametrize("variant", [0, 3])
@pytest.mark.parametrize("M,N,K", [(8192, 3072, 768), (8192, 768, 3072), (16384, 6144, 4096), (16384, 4096, 4096),
                                   (16384, 28672, 4096), (16384, 4096, 14336)])
def test_model_shapes_sampled(nv, variant, M, N, K):
    """GPT-2-small MLP and all four Llama-3-8B linear shapes at full size against the oracle on a sample that holds
    the first and last row of every 128- and 256-row tile and the first and last column of every 128-, 192- and
    256-column tile (every tile band edge of every kernel variant) plus random interior points, and linearity in
    alpha (a size-independent property)."""
    nv.set_gemm_variant(variant)
    g = torch.Generator("cuda").manual_seed(3456)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    y = nv.gemm(xc, xs, wc, ws)
    nv.check_status()
    gi = torch.Generator().manual_seed(7)
    rows = band_edge_samples(M, (128, 256), 32, gi)
    cols = band_edge_samples(N, (128, 192, 256), 32, gi)
    ref = oracle_gemm(nv, x, w, rows=rows.numpy(), cols=cols.numpy())
    assert_close(y[rows.cuda()][:, cols.cuda()].cpu(), ref)
    y2 = nv.gemm(xc, xs, wc, ws, alpha=2.0)
    assert torch.equal((y.float() * 2).bfloat16().view(torch.int16), y2.view(torch.int16))   # exact: power-of-two alpha


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("splits", [2, 3, 8])
def test_split_k_forced(nv, variant, splits):
    """K divided among work units, fp32 partial sums in the workspace, second-pass reduction."""
    nv.set_gemm_variant(variant, splits=splits)
    try:
        run(nv, 384, 512, 2048, alpha=0.5, beta=2.0, use_bias=True)
        run(nv, 300, 200, 1152)                 # ragged tiles; 9 k-blocks do not divide by 2 or 8
        run(nv, 130, 100, 640)                  # N % 4 != 0: scalar partial stores and reduction
    finally:
        nv.set_gemm_variant(0)


def test_split_k_automatic_for_weight_gradient_shapes(nv, native_lib):
    """Small outputs with a long contraction (weight gradients of narrow layers over many tokens): the
    planner splits K when the tiles would occupy less than a quarter of the GPU."""
    nv.set_gemm_variant(0)
    assert native_lib.dw_mxfp8_gemm_workspace(1024, 1024, 16384) == 4 * 1024 * 1024 * 4
    assert native_lib.dw_mxfp8_gemm_workspace(3072, 768, 8192) == 0        # GPT-2-small wgrad: half the GPU, unsplit
    assert native_lib.dw_mxfp8_gemm_workspace(16384, 4096, 4096) == 0
    run(nv, 1024, 1024, 16384)
    run(nv, 3072, 768, 8192)
    run(nv, 768, 3072, 8192)
    # same operands, split and unsplit, agree to bf16 rounding of the same fp32 sums
    g = torch.Generator("cpu").manual_seed(5)
    a = torch.randn(768, 16384, generator=g).bfloat16().cuda()
    b = torch.randn(1024, 16384, generator=g).bfloat16().cuda()
    ac, asf = nv.quantize(a, nv.DIR_ROW, 0, nv.SF_TILED)
    bc, bsf = nv.quantize(b, nv.DIR_ROW, 0, nv.SF_TILED)
    y_split = nv.gemm(ac, asf, bc, bsf)
    nv.set_gemm_variant(0, splits=1)
    y_one = nv.gemm(ac, asf, bc, bsf)
    nv.set_gemm_variant(0)
    nv.check_status()
    assert_close(y_split.cpu(), y_one.float().cpu())


def test_backward_operand_forms(nv):
    """dgrad and wgrad through column-wise (transposed) operands: contraction over N and over M."""
    nv.set_gemm_variant(0)
    M, N, K = 512, 384, 256
    g = torch.Generator("cpu").manual_seed(11)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    dy = torch.randn(M, N, generator=g).bfloat16().cuda()
    dyr, dyrs, dyc, dycs = nv.quantize_both(dy, 0, nv.SF_TILED)
    _, _, wct, wcs = nv.quantize_both(w, 0, nv.SF_TILED)
    _, _, xct, xcs = nv.quantize_both(x, 0, nv.SF_TILED)
    dx = nv.gemm(dyr, dyrs, wct, wcs)            # [M, K], contraction N
    dw = nv.gemm(dyc, dycs, xct, xcs)            # [N, K], contraction M
    nv.check_status()
    ref_dx = oracle_gemm(nv, dy, w.t().contiguous())
    ref_dw = oracle_gemm(nv, dy.t().contiguous(), x.t().contiguous())
    assert_close(dx.cpu(), ref_dx)
    assert_close(dw.cpu(), ref_dw)


def test_zero_and_nan_free_padding(nv):
    """Ragged M/N/K tiles: out-of-range operand rows are zero-filled and padding scales are finite,
    so no NaN leaks into valid outputs; an all-zero operand gives exact zeros."""
    nv.set_gemm_variant(0)
    x = torch.zeros(130, 96, dtype=torch.bfloat16, device="cuda")
    w = torch.randn(70, 96, device="cuda").bfloat16()
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    # the caller's scale buffers may hold anything beyond what the quantiser wrote: poison D first
    out = torch.full((130, 70), float("nan"), dtype=torch.bfloat16, device="cuda")
    y = nv.gemm(xc, xs, wc, ws, out=out)
    nv.check_status()
    assert torch.count_nonzero(y).item() == 0


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "silu"])
@pytest.mark.parametrize("shape", [(384, 512, 256), (300, 160, 96)])
def test_fused_epilogue_activation_and_quantised_output(nv, act, shape):
    """dw_mxfp8_gemm_fused: D = act(A.B^T + bias) within tolerance of the fp32 reference, and the quantised
    output is bit-for-bit what the row-wise quantiser gives on that D (codes, scales, padding bytes)."""
    nv.set_gemm_variant(0)
    M, N, K = shape
    g = torch.Generator("cpu").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    d, codes, scales = nv.gemm_fused(xc, xs, wc, ws, bias=bias, activation=act)
    nv.check_status()
    pre = oracle_gemm(nv, x, w, bias=bias)
    fn = {"none": lambda t: t, "relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu}[act]
    assert_close(d.cpu(), fn(pre))
    bits = d.cpu().view(torch.int16).numpy().view(np.uint16)
    ec, es = o.quantize_rowwise(bits)
    assert np.array_equal(host(codes), ec)
    assert np.array_equal(host(scales), o.sf_flat_to_tiled(es))
    # quantised form only (no bf16 D written): same bytes
    d2, codes2, scales2 = nv.gemm_fused(xc, xs, wc, ws, bias=bias, activation=act, write_d=False)
    nv.check_status()
    assert d2 is None and torch.equal(codes2.view(torch.uint8), codes.view(torch.uint8)) and torch.equal(scales2, scales)


@pytest.mark.parametrize("shape", [(384, 512, 256), (300, 320, 96), (129, 1024 + 64, 160), (2048, 2048, 512)])
@pytest.mark.parametrize("variant", [0, 2, 3])
def test_swiglu_epilogue(nv, shape, variant):
    """dw_mxfp8_gemm_fused(DW_ACT_SWIGLU): gate and up rows interleaved in groups of 32, h = silu(gate) * up formed from
    the fp32 accumulators.  The bf16 h is within the GEMM tolerance of silu(g) * u computed from the oracle's fp32 GEMM,
    and the quantised output (codes, tiled scales, padding bytes) is bit for bit the oracle's row-wise quantisation of
    that bf16 h, with and without the bf16 copy being written.  Shapes cover ragged row tiles, F not a multiple of 128
    (padded scale k-blocks) and several column tiles; variants the single-CTA and the CTA-pair kernel."""
    M, F2, K = shape
    Fh = F2 // 2
    nv.set_gemm_variant(variant)
    g = torch.Generator("cpu").manual_seed(M + F2 + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    wg = (torch.randn(Fh, K, generator=g) * 0.1).bfloat16().cuda()
    wu = (torch.randn(Fh, K, generator=g) * 0.1).bfloat16().cuda()
    w = nv.interleave_gate_up(wg, wu).contiguous()
    assert torch.equal(w[:32], wg[:32]) and torch.equal(w[32:64], wu[:32]) and torch.equal(w[64:96], wg[32:64])
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    h, codes, scales = nv.gemm_fused(xc, xs, wc, ws, activation="swiglu")
    nv.check_status()
    nv.set_gemm_variant(0)
    assert h.shape == (M, Fh) and codes.shape == (M, Fh)
    gate, up = oracle_gemm(nv, x, wg), oracle_gemm(nv, x, wu)
    assert_close(h.cpu(), torch.nn.functional.silu(gate) * up)
    bits = h.cpu().view(torch.int16).numpy().view(np.uint16)
    ec, es = o.quantize_rowwise(bits)
    assert np.array_equal(host(codes), ec)
    assert np.array_equal(host(scales), o.sf_flat_to_tiled(es))
    nv.set_gemm_variant(variant)
    h2, codes2, scales2 = nv.gemm_fused(xc, xs, wc, ws, activation="swiglu", write_d=False)
    nv.check_status()
    nv.set_gemm_variant(0)
    assert h2 is None and torch.equal(codes2.view(torch.uint8), codes.view(torch.uint8)) and torch.equal(scales2, scales)
    # per-thread stores instead of TMA stores for the bf16 copy: same bits
    nv.set_gemm_variant(variant, direct_stores=True)
    h3, _, _ = nv.gemm_fused(xc, xs, wc, ws, activation="swiglu", quantize_out=False)
    nv.check_status()
    nv.set_gemm_variant(0)
    assert torch.equal(h3.view(torch.int16), h.view(torch.int16))


def test_swiglu_rejects_bad_arguments(nv, native_lib):
    p16 = 16
    L = native_lib
    args = (p16, p16, p16, p16, p16, None, 128, 96, 128, 1.0)
    assert L.dw_mxfp8_gemm_fused(*args, 0.0, 4, None, None, 0, None, None) == -1        # fused width not a multiple of 64
    args = (p16, p16, p16, p16, p16, None, 128, 128, 128, 1.0)
    assert L.dw_mxfp8_gemm_fused(*args, 1.0, 4, None, None, 0, None, None) == -1        # beta with the gated epilogue
    assert L.dw_mxfp8_gemm_fused(*args, 0.0, 5, None, None, 0, None, None) == -1        # no such activation


def test_fused_mlp_chain_never_stores_the_activation(nv):
    """up-projection with bias + GELU + quantise fused, then the down-projection consumes the codes directly:
    identical bits to GEMM -> bf16 -> quantise -> GEMM."""
    nv.set_gemm_variant(0)
    g = torch.Generator("cpu").manual_seed(9)
    x = torch.randn(512, 256, generator=g).bfloat16().cuda()
    w1 = (torch.randn(1024, 256, generator=g) * 0.06).bfloat16().cuda()
    b1 = torch.randn(1024, generator=g).bfloat16().cuda()
    w2 = (torch.randn(256, 1024, generator=g) * 0.03).bfloat16().cuda()
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    w1c, w1s = nv.quantize(w1, nv.DIR_ROW, 0, nv.SF_TILED)
    w2c, w2s = nv.quantize(w2, nv.DIR_ROW, 0, nv.SF_TILED)
    _, hc, hs = nv.gemm_fused(xc, xs, w1c, w1s, bias=b1, activation="gelu", write_d=False)
    y_fused = nv.gemm(hc, hs, w2c, w2s)
    h, _, _ = nv.gemm_fused(xc, xs, w1c, w1s, bias=b1, activation="gelu", quantize_out=False)
    hc2, hs2 = nv.quantize(h, nv.DIR_ROW, 0, nv.SF_TILED)
    y_two = nv.gemm(hc2, hs2, w2c, w2s)
    nv.check_status()
    assert torch.equal(y_fused.view(torch.int16), y_two.view(torch.int16))
    ref = torch.nn.functional.gelu(x.float() @ w1.float().t() + b1.float()) @ w2.float().t()
    # sanity against unquantised fp32: E4M3 keeps 3 mantissa bits, so two quantised layers sit near 5 % (Frobenius)
    assert ((y_fused.float() - ref).norm() / ref.norm()).item() < 0.08


@pytest.mark.parametrize("sizes", [[300, 0, 128, 1, 700], [2048, 1024, 4096, 512], [64, 64, 64, 64, 64, 64, 64, 64]])
def test_grouped_gemm_one_launch_equals_one_gemm_per_group(nv, sizes):
    """dw_mxfp8_gemm_grouped (the experts of an MoE layer in one launch) against the ordinary GEMM run once per
    group: same kernel and accumulation order, so the bf16 outputs are identical; one group also goes to the oracle.
    Sizes cover an empty group, a one-row group, ragged groups and both row-tile granularities (128, 256)."""
    from deepwell_b200 import cutlass_kernels as ck
    K, N = 512, 384
    g = torch.Generator("cpu").manual_seed(sum(sizes))
    a_list = [torch.randn(m, K, generator=g).bfloat16().cuda() for m in sizes]
    w_list = [(torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda() for _ in sizes]       # [N, K] weights
    nv.set_gemm_variant(0)
    got = ck.mxfp8_grouped_gemm_bf16(a_list, [w.t() for w in w_list], alpha=0.5)
    nv.check_status()
    assert [tuple(o.shape) for o in got] == [(m, N) for m in sizes]
    for variant in (2, 3):            # the grouped launch uses the 1-CTA kernel for 128-row tiles, the CTA pair for 256
        nv.set_gemm_variant(variant)
        for a, w, o_ in zip(a_list, w_list, got):
            if a.shape[0] == 0:
                continue
            ref = ck.mxfp8_gemm_bf16(a, w.t(), None, 0.5, 0.0)
            assert torch.equal(ref.view(torch.int16), o_.view(torch.int16))
    nv.set_gemm_variant(0)
    big = max(range(len(sizes)), key=lambda i: sizes[i])
    assert_close(got[big].cpu(), oracle_gemm(nv, a_list[big], w_list[big], alpha=0.5))


def test_grouped_gemm_rejects_bad_arguments(nv, native_lib):
    p16 = 16
    L = native_lib
    assert L.dw_mxfp8_gemm_grouped(p16, p16, p16, p16, p16, p16, 300, 128, 128, 2, 256, 1.0, None, None) == -1   # M not whole tiles
    assert L.dw_mxfp8_gemm_grouped(p16, p16, p16, p16, p16, p16, 512, 96, 128, 2, 256, 1.0, None, None) == -1    # N % 128
    assert L.dw_mxfp8_gemm_grouped(p16, p16, p16, p16, p16, p16, 512, 128, 128, 2, 192, 1.0, None, None) == -1   # tile height
    assert L.dw_mxfp8_gemm_grouped(p16, p16, p16, p16, p16, None, 512, 128, 128, 2, 256, 1.0, None, None) == -1  # no tile_group


def test_grouped_gemm_weight_cache_and_quantize_into(nv):
    """Repeated grouped calls with unchanged weights reuse the stacked operand; an in-place weight update is seen.
    quantize_into writes one expert's slice of a stacked operand exactly as quantize would."""
    from deepwell_b200 import cutlass_kernels as ck
    K, N, G = 256, 256, 3
    g = torch.Generator("cpu").manual_seed(99)
    a_list = [torch.randn(m, K, generator=g).bfloat16().cuda() for m in (200, 56, 384)]
    w_list = [(torch.randn(K, N, generator=g) * 0.05).bfloat16().cuda() for _ in range(G)]      # [K, N]: column-wise path
    cache = {}
    first = ck.mxfp8_grouped_gemm_bf16(a_list, w_list, weight_cache=cache)
    operand = cache["operand"][0]
    again = ck.mxfp8_grouped_gemm_bf16(a_list, w_list, weight_cache=cache)
    assert cache["operand"][0] is operand
    for x, y in zip(first, again):
        assert torch.equal(x, y)
    w_list[1].mul_(2.0)
    third = ck.mxfp8_grouped_gemm_bf16(a_list, w_list, weight_cache=cache)
    assert cache["operand"][0] is not operand
    limit, ck._STACK_LIMIT = ck._STACK_LIMIT, 0           # the path for large experts: one quantiser launch per expert
    try:
        for mixed in (w_list, [w_list[0], w_list[1].t().contiguous().t(), w_list[2]]):     # [K, N] and K-major views
            per_expert = ck.mxfp8_grouped_gemm_bf16(a_list, mixed)
            for x, y in zip(third, per_expert):
                assert torch.equal(x, y)
    finally:
        ck._STACK_LIMIT = limit
    assert torch.equal(third[1].view(torch.int16), (first[1].float() * 2).bfloat16().view(torch.int16))    # exact: power of two
    assert torch.equal(third[0], first[0]) and torch.equal(third[2], first[2])
    # quantize_into == quantize
    x = torch.randn(N, K, generator=g).bfloat16().cuda()
    codes, scales = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    big_c = torch.zeros(3 * N, K, dtype=torch.uint8, device="cuda")
    big_s = torch.zeros(3 * scales.numel(), dtype=torch.uint8, device="cuda")
    nv.quantize_into(x, big_c[N:2 * N], big_s[scales.numel():2 * scales.numel()], nv.DIR_ROW, 0, nv.SF_TILED)
    assert torch.equal(big_c[N:2 * N], codes.view(torch.uint8)) and torch.equal(big_s[scales.numel():2 * scales.numel()], scales)
    assert int(big_c[:N].sum()) == 0 and int(big_c[2 * N:].sum()) == 0


# ----------------------------------------------------------------------------------------------
# the boundary: plan per call, host threads, tensor-map table, error paths
# ----------------------------------------------------------------------------------------------
def test_two_host_threads_two_streams_two_variants(nv, native_lib):
    """Two host threads, each on its own stream, run the block-scaled GEMM with DIFFERENT kernel variants (passed per
    call as the plan word) and the tile quantiser at the same time; both get oracle-correct results, repeatedly.
    Nothing a call reads is process state, so neither thread can change what the other runs."""
    import threading
    nv.set_gemm_variant(0)
    L = native_lib
    M, N, K = 640, 768, 1024
    g = torch.Generator("cpu").manual_seed(21)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.03).bfloat16().cuda()
    ref = oracle_gemm(nv, x, w)
    e_r, e_rs = o.quantize_rowwise(x.cpu().view(torch.int16).numpy().view(np.uint16))
    e_c, e_cs = o.quantize_colwise(x.cpu().view(torch.int16).numpy().view(np.uint16))
    status = nv.status_word("cuda:0")
    torch.cuda.synchronize()
    errors, results = [], {}

    def worker(name, variant):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device="cuda")
                for it in range(6):
                    cr, ct = u8(M, K), u8(K, M)
                    sr, sc = u8(nv.scale_bytes(M, K, nv.SF_TILED)), u8(nv.scale_bytes(K, M, nv.SF_TILED))
                    rc = L.dw_mxfp8_quantize_both(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), ct.data_ptr(), sc.data_ptr(), M, K,
                                                  0, nv.SF_TILED, stream.cuda_stream)
                    assert rc == 0
                    wc, ws = u8(N, K), u8(nv.scale_bytes(N, K, nv.SF_TILED))
                    assert L.dw_mxfp8_quantize(w.data_ptr(), wc.data_ptr(), ws.data_ptr(), N, K, 0, 0, nv.SF_TILED, stream.cuda_stream) == 0
                    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
                    rc = L.dw_mxfp8_gemm_planned(cr.data_ptr(), sr.data_ptr(), wc.data_ptr(), ws.data_ptr(), y.data_ptr(), None,
                                                 M, N, K, 1.0, 0.0, None, 0, nv.plan_word(variant), status.data_ptr(),
                                                 stream.cuda_stream)
                    assert rc == 0
                    stream.synchronize()
                    results[(name, it)] = (y.cpu(), cr.cpu().numpy(), sr.cpu().numpy(), ct.cpu().numpy(), sc.cpu().numpy())
        except Exception as e:          # surfaced in the main thread
            errors.append((name, repr(e)))

    threads = [threading.Thread(target=worker, args=("pair", 3)), threading.Thread(target=worker, args=("single", 2))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    nv.check_status()
    for (name, it), (y, cr, sr, ct, sc) in results.items():
        assert_close(y, ref)
        assert np.array_equal(cr, e_r) and np.array_equal(sr, o.sf_flat_to_tiled(e_rs)), (name, it)
        assert np.array_equal(ct, e_c) and np.array_equal(sc, o.sf_flat_to_tiled(e_cs)), (name, it)
    # the two variants really are different kernels with the same result up to accumulation order: compare one pair
    assert_close(results[("pair", 0)][0], results[("single", 0)][0].float())


def test_kernel_objects_keep_their_own_cluster_shape(nv):
    """set_cluster_shape on one BlackwellGemmKernel pins that object only; another object and the process default are
    untouched (the choice travels with each call as its plan word)."""
    from deepwell_b200 import cutlass_kernels as ck
    nv.set_gemm_variant(0)
    a = torch.randn(512, 256, device="cuda").bfloat16()
    b = (torch.randn(256, 384, device="cuda") * 0.05).bfloat16()
    k1, k2 = ck.BlackwellGemmKernel(), ck.BlackwellGemmKernel()
    for k in (k1, k2):
        k.initialize(512, 384, 256, "mxfp8", True, 32)
    k1.set_cluster_shape(1, 1)
    assert k1.plan == nv.plan_word(2) and k2.plan == nv.plan_word(0) and k2.cluster_shape is None
    y1, y2 = k1.gemm(a, b), k2.gemm(a, b)
    nv.check_status()
    ref = oracle_gemm(nv, a, b.t().contiguous())
    assert_close(y1.cpu(), ref)
    assert_close(y2.cpu(), ref)


def test_tensor_maps_are_encoded_once_per_buffer(nv, native_lib):
    """A second GEMM on the same buffers encodes no tensor map (they come from the per-thread table); new buffers do."""
    nv.set_gemm_variant(0)
    x = torch.randn(384, 256, device="cuda").bfloat16()
    w = torch.randn(512, 256, device="cuda").bfloat16()
    xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
    wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
    out = torch.empty(384, 512, dtype=torch.bfloat16, device="cuda")
    first = nv.gemm(xc, xs, wc, ws, out=out).clone()
    n0 = native_lib.dw_mxfp8_debug_counter(0)
    again = nv.gemm(xc, xs, wc, ws, out=out)
    assert native_lib.dw_mxfp8_debug_counter(0) == n0
    assert torch.equal(first, again)
    out2 = torch.empty(384, 512, dtype=torch.bfloat16, device="cuda")
    nv.gemm(xc, xs, wc, ws, out=out2)
    assert native_lib.dw_mxfp8_debug_counter(0) == n0 + 1          # only the output map is new
    assert torch.equal(first, out2)
    nv.check_status()


def test_status_word_set_from_the_host_raises(nv):
    """The error path above the kernels, without a device fault: a non-zero status word (here written by the host,
    as a kernel whose wait expired would) makes check_status raise a RuntimeError that names the wait and the CTA,
    and clears the word."""
    sw = nv.status_word("cuda:0")
    sw.fill_(3 | (17 << 8))                      # code 3 (accumulator wait) recorded by CTA 17
    with pytest.raises(RuntimeError, match=r"status word 3, CTA 17"):
        nv.check_status("cuda:0")
    assert int(sw.item()) == 0
    nv.check_status("cuda:0")                    # clean again


def test_bounded_wait_runs_out_and_is_reported(nv, native_lib):
    """A wait that nothing satisfies gives up after its limit (100 000 cycles here, ~50 us), the kernel returns, the
    status word carries its code and the C ABI reports DW_ERR_DEVICE_STATUS; the context stays usable.  The kernel
    is the library's self-test: one thread on an mbarrier nobody arrives at, no copy or tensor-core work in flight."""
    L = native_lib
    sw = nv.status_word("cuda:0")
    sw.zero_()
    st = torch.cuda.current_stream().cuda_stream
    assert L.dw_mxfp8_selftest_bounded_wait(100000, sw.data_ptr(), st) == 0
    assert L.dw_mxfp8_check_status(sw.data_ptr(), st) == -4
    assert int(sw.item()) == 5                   # self-test code, CTA 0
    with pytest.raises(RuntimeError, match=r"status word 5, CTA 0"):
        nv.check_status("cuda:0")
    # the context is intact: a GEMM right after gives the right answer
    run(nv, 256, 256, 256)
