"""GPU parity tests of the MX quantiser: CUDA kernels (through the C ABI) against the oracle.
Bar: bit-exact codes and scales."""
import hashlib

import numpy as np
import pytest
import torch

from conftest import config1_inputs
from oracle import mx_oracle as o
from oracle import mx_ref as c

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nv(native_lib):
    from deepwell_b200 import _native
    assert torch.cuda.is_available(), "the parity tests need a GPU"
    assert native_lib.dw_mxfp8_device_supported(0) == 1, "sm_100a device required"
    return _native


def bits_of(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()


def host(t):
    return t.view(torch.uint8).cpu().numpy()


def check_all_forms(nv, x, rule):
    """Every direction and both scale layouts of one input against the C restatement."""
    xb = bits_of(x)
    er, ers = c.quantize_rowwise(xb, rule)
    et, ets = c.quantize_colwise(xb, rule, True)
    en, _ = c.quantize_colwise(xb, rule, False)
    for layout in (nv.SF_FLAT, nv.SF_TILED):
        exp_rs = ers if layout == nv.SF_FLAT else o.sf_flat_to_tiled(ers)
        exp_ts = ets if layout == nv.SF_FLAT else o.sf_flat_to_tiled(ets)
        gc, gs = nv.quantize(x, nv.DIR_ROW, rule, layout)
        assert np.array_equal(host(gc), er) and np.array_equal(host(gs).reshape(exp_rs.shape), exp_rs)
        gc, gs = nv.quantize(x, nv.DIR_COL_T, rule, layout)
        assert np.array_equal(host(gc), et) and np.array_equal(host(gs).reshape(exp_ts.shape), exp_ts)
        gc, gs = nv.quantize(x, nv.DIR_COL, rule, layout)
        assert np.array_equal(host(gc), en) and np.array_equal(host(gs).reshape(exp_ts.shape), exp_ts)
        a, b, cc, d = nv.quantize_both(x, rule, layout)
        assert np.array_equal(host(a), er) and np.array_equal(host(b).reshape(exp_rs.shape), exp_rs)
        assert np.array_equal(host(cc), et) and np.array_equal(host(d).reshape(exp_ts.shape), exp_ts)


@pytest.mark.parametrize("rule", [0, 1])
def test_kat_vectors(nv, golden, rule):
    k = golden["kat_quant"]
    name = o.SCALE_RULES[rule]
    x = from_bits(k["bits"])
    gc, gs = nv.quantize(x, nv.DIR_ROW, rule, nv.SF_FLAT)
    assert np.array_equal(host(gc), k[f"row_codes_{name}"]) and np.array_equal(host(gs), k[f"row_scales_{name}"])
    gc, gs = nv.quantize(x, nv.DIR_COL_T, rule, nv.SF_FLAT)
    assert np.array_equal(host(gc), k[f"col_codes_{name}"]) and np.array_equal(host(gs), k[f"col_scales_{name}"])
    check_all_forms(nv, x, rule)


@pytest.mark.parametrize("shape", [(128, 128), (256, 512), (96, 160), (32, 96), (33, 64), (1, 32), (7, 50), (129, 4096),
                                   (4096, 128), (300, 1000), (1, 1), (31, 31), (64, 8), (2048, 1024),
                                   (2048 + 3, 1024 + 32), (1031, 2080)])     # the last two: the large-input row kernel, ragged slabs
@pytest.mark.parametrize("rule", [0, 1])
def test_shapes_fast_and_ragged(nv, shape, rule):
    g = torch.Generator("cpu").manual_seed(shape[0] * 7919 + shape[1])
    x = torch.randn(shape, generator=g)
    x[torch.rand(shape, generator=g) < 0.01] *= 50
    check_all_forms(nv, x.bfloat16().cuda(), rule)


@pytest.mark.parametrize("shape", [(128, 128), (256, 512), (96, 160), (32, 96), (2048, 1024), (4096, 128), (160, 96)])
@pytest.mark.parametrize("one_group", [4, 8])
def test_staged_transposed_write_out_gives_the_same_bytes(nv, shape, one_group):
    """The column-wise kernel's staged write-out (the default) and the direct one (tuning word 1), whole and ragged
    tiles, with the fused kernel's two passes run by one group of threads one after the other (tuning bit 2) and by two
    groups side by side (bit 3; what large inputs get): every form still equals the C restatement."""
    g = torch.Generator("cpu").manual_seed(shape[0] * 31 + shape[1])
    x = torch.randn(shape, generator=g)
    x[torch.rand(shape, generator=g) < 0.01] *= 50
    x = x.bfloat16().cuda()
    L = nv.load()
    assert L.dw_mxfp8_quantize_set_tuning(2 | one_group) == 0
    try:
        check_all_forms(nv, x, 0)
        if shape[0] % 32 == 0 and shape[1] % 32 == 0:
            a = nv.quantize_both_colsum(x, 0, nv.SF_TILED)
            assert L.dw_mxfp8_quantize_set_tuning(1 | one_group) == 0          # the direct write-out
            check_all_forms(nv, x, 0)
            b = nv.quantize_both_colsum(x, 0, nv.SF_TILED)
            for u, v in zip(a, b):
                assert torch.equal(u.view(torch.uint8) if u.element_size() == 1 else u, v.view(torch.uint8) if v.element_size() == 1 else v)
    finally:
        assert L.dw_mxfp8_quantize_set_tuning(0) == 0
    assert L.dw_mxfp8_quantize_set_tuning(3) == -1 and L.dw_mxfp8_quantize_set_tuning(32) == -1 and L.dw_mxfp8_quantize_set_tuning(12) == -1
    assert L.dw_mxfp8_quantize_set_tuning(4) == 0 and L.dw_mxfp8_quantize_set_tuning(0) == 0


@pytest.mark.parametrize("shape", [(128, 128), (4096, 1024), (96, 160), (8192, 3072), (2048, 14336 + 32)])
def test_column_kernel_with_two_and_three_tile_buffers_gives_the_same_bytes(nv, shape):
    """The column-wise kernel keeps two tiles in flight (three tile buffers, the default up to 2^28 elements) or one (two
    buffers, tuning bit 4): the same bytes, equal to the C restatement; with more tiles than thread blocks, so that the
    ring of buffers wraps several times, and with a ragged last tile."""
    g = torch.Generator("cpu").manual_seed(shape[0] + shape[1])
    x = torch.randn(shape, generator=g)
    x[torch.rand(shape, generator=g) < 0.01] *= 50
    x = x.bfloat16().cuda()
    L = nv.load()
    et, ets = c.quantize_colwise(bits_of(x), 0, True)
    exp_ts = o.sf_flat_to_tiled(ets)
    try:
        for word in (0, 16):
            assert L.dw_mxfp8_quantize_set_tuning(word) == 0
            gc, gs = nv.quantize(x, nv.DIR_COL_T, 0, nv.SF_TILED)
            assert np.array_equal(host(gc), et) and np.array_equal(host(gs).reshape(exp_ts.shape), exp_ts)
    finally:
        assert L.dw_mxfp8_quantize_set_tuning(0) == 0


def test_every_bf16_pattern(nv):
    """NaN, Inf, subnormals, signed zeros: all 65536 patterns, shuffled, both directions and rules."""
    bits = np.random.default_rng(1).permutation(65536).astype(np.uint16).reshape(512, 128)
    for rule in (0, 1):
        check_all_forms(nv, from_bits(bits), rule)


def test_empty_inputs(nv):
    for shape in [(0, 64), (64, 0)]:
        x = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
        codes, scales = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_FLAT)
        assert codes.numel() == 0


def test_unaligned_views_take_the_generic_path(nv):
    base = torch.randn(257 * 96 + 1, device="cuda").bfloat16()
    x = base[1:].view(257, 96)                      # 2-byte aligned only
    assert x.data_ptr() % 16 != 0
    xb = bits_of(x)
    L = nv.load()
    codes = torch.empty(257, 96, dtype=torch.uint8, device="cuda")
    scales = torch.empty(257 * 3, dtype=torch.uint8, device="cuda")
    rc = L.dw_mxfp8_quantize(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), 257, 96, 0, 0, 0,
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    er, ers = c.quantize_rowwise(xb, 0)
    assert np.array_equal(codes.cpu().numpy(), er) and np.array_equal(scales.cpu().numpy().reshape(ers.shape), ers)


def test_config1_against_golden_digests(nv, golden):
    g = golden["config1"]
    X, W = config1_inputs()
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    xc, xs = nv.quantize(X.cuda(), nv.DIR_ROW, 0, nv.SF_FLAT)
    wc, ws = nv.quantize(W.cuda(), nv.DIR_ROW, 0, nv.SF_FLAT)
    assert sha(host(xc)) == str(g["x_codes_sha"]) and sha(host(xs)) == str(g["x_scales_sha"])
    assert sha(host(wc)) == str(g["w_codes_sha"]) and sha(host(ws)) == str(g["w_scales_sha"])
    assert np.array_equal(host(xc)[:8, :64], g["x_codes_head"])


def test_dequantize_matches_oracle(nv):
    x = (torch.randn(256, 512) * 3).bfloat16().cuda()
    for layout in (nv.SF_FLAT, nv.SF_TILED):
        gc, gs = nv.quantize(x, nv.DIR_ROW, 0, layout)
        dq = nv.dequantize(gc, gs, layout)
        fc, fs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_FLAT)
        exp = o.f32_to_bf16_bits(o.dequantize_rowwise(host(fc), host(fs)))
        assert np.array_equal(bits_of(dq), exp)
    x = torch.randn(5, 50).bfloat16().cuda()           # ragged: scalar path
    gc, gs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_FLAT)
    exp = o.f32_to_bf16_bits(o.dequantize_rowwise(host(gc), host(gs)))
    assert np.array_equal(bits_of(nv.dequantize(gc, gs, nv.SF_FLAT)), exp)


@pytest.mark.parametrize("rows,cols", [(16384, 4096), (16384, 14336), (1 << 21, 128), (4096, 16384)])
def test_full_size_properties(nv, rows, cols):
    """At BASELINE sizes (Student-t(3) x 0.5 inputs): sampled row blocks against the oracle, the
    column-wise payload equals the row-wise payload of the transpose, idempotence of
    quantise(dequantise(q)), and the fused kernel equals the two single-direction kernels."""
    g = torch.Generator("cuda").manual_seed(4567)
    z = torch.randn(rows, cols, device="cuda", generator=g)
    v = torch.distributions.Chi2(torch.tensor(3.0, device="cuda")).sample((rows, 1))
    x = (0.5 * z / torch.sqrt(v / 3)).bfloat16()
    del z
    rc, rs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_FLAT)
    sel = torch.randint(0, rows, (64,), generator=torch.Generator().manual_seed(1)).tolist()
    er, ers = c.quantize_rowwise(bits_of(x[sel]), 0)
    assert np.array_equal(host(rc[sel]), er) and np.array_equal(host(rs[sel]), ers)
    tc, ts = nv.quantize(x, nv.DIR_COL_T, 0, nv.SF_FLAT)
    xt = x.t().contiguous()
    tc2, ts2 = nv.quantize(xt, nv.DIR_ROW, 0, nv.SF_FLAT)
    assert torch.equal(tc.view(torch.uint8), tc2.view(torch.uint8)) and torch.equal(ts, ts2)
    del xt, tc2, ts2
    a, b, cc, d = nv.quantize_both(x, 0, nv.SF_FLAT)
    assert torch.equal(a.view(torch.uint8), rc.view(torch.uint8)) and torch.equal(b, rs)
    assert torch.equal(cc.view(torch.uint8), tc.view(torch.uint8)) and torch.equal(d, ts)
    dq = nv.dequantize(rc, rs, nv.SF_FLAT)
    rc2, rs2 = nv.quantize(dq, nv.DIR_ROW, 0, nv.SF_FLAT)
    dq2 = nv.dequantize(rc2, rs2, nv.SF_FLAT)
    assert torch.equal(dq.view(torch.int16), dq2.view(torch.int16))      # idempotent after one round trip


def test_largest_sweep_point_2_pow_32_elements(nv):
    """The top of the quantise sweep (2^32 elements, K = 16384): 64-bit addressing everywhere.  Row blocks
    sampled from the start, the middle and the very end against the oracle; column-wise payload of
    sampled columns against the oracle on the gathered columns."""
    rows, cols = 1 << 18, 1 << 14
    x = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    g = torch.Generator("cuda").manual_seed(4567)
    for r0 in range(0, rows, 1 << 14):                      # filled in slices: no 16 GiB fp32 temporary
        z = torch.randn(1 << 14, cols, device="cuda", generator=g)
        v = torch.distributions.Chi2(torch.tensor(3.0, device="cuda")).sample((1 << 14, 1))
        x[r0:r0 + (1 << 14)] = (0.5 * z / torch.sqrt(v / 3)).bfloat16()
    del z, v
    rc, rs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_FLAT)
    sel = [0, 1, 131071, 131072, rows - 2, rows - 1]
    er, ers = c.quantize_rowwise(bits_of(x[sel]), 0)
    assert np.array_equal(host(rc[sel]), er) and np.array_equal(host(rs[sel]), ers)
    del rc, rs
    tc, ts = nv.quantize(x, nv.DIR_COL_T, 0, nv.SF_FLAT)
    csel = [0, 77, cols - 1]
    xs = x[:, csel].t().contiguous()                        # [3, rows]: the sampled columns as rows
    ec, ecs = c.quantize_rowwise(bits_of(xs), 0)
    assert np.array_equal(host(tc[csel]), ec) and np.array_equal(host(ts[csel]), ecs)


@pytest.mark.parametrize("rows,cols", [(32, 32), (160, 96), (4096, 768), (8192, 3072), (1000 * 32, 128)])
def test_quantize_both_with_column_sums(nv, rows, cols):
    """dw_mxfp8_quantize_both_colsum: the four quantised outputs are those of dw_mxfp8_quantize_both bit for bit;
    the column sums match a float64 sum within fp32 accumulation error (tolerance: 1e-5 x the column's sum of
    magnitudes, plus bf16 rounding of the result in bf16 mode), and two calls give identical bits."""
    g = torch.Generator("cuda").manual_seed(rows * 7 + cols)
    x = torch.randn(rows, cols, device="cuda", generator=g)
    x[torch.rand(rows, cols, device="cuda", generator=g) < 0.01] *= 50
    x = (x + 0.25).bfloat16()                     # non-zero mean so that the sums do not cancel to nothing
    ref4 = nv.quantize_both(x, 0, nv.SF_TILED)
    got = nv.quantize_both_colsum(x, 0, nv.SF_TILED, out_dtype=torch.float32)
    again = nv.quantize_both_colsum(x, 0, nv.SF_TILED, out_dtype=torch.float32)
    for a, b in zip(ref4, got[:4]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert torch.equal(got[4].view(torch.int32), again[4].view(torch.int32))
    exact = x.double().sum(0)
    bound = 1e-5 * x.double().abs().sum(0) + 1e-30
    assert ((got[4].double() - exact).abs() <= bound).all()
    as_bf16 = nv.quantize_both_colsum(x, 0, nv.SF_TILED, out_dtype=torch.bfloat16)[4]
    assert as_bf16.dtype == torch.bfloat16
    assert torch.equal(as_bf16.view(torch.int16), got[4].bfloat16().view(torch.int16))


def test_column_sums_reject_shapes_outside_the_tile_kernel(nv, native_lib):
    x = torch.zeros(48, 40, dtype=torch.bfloat16, device="cuda")
    p = x.data_ptr()
    rc = native_lib.dw_mxfp8_quantize_both_colsum(p, p, p, p, p, 48, 40, 0, 1, p, 0, p, 1 << 20, None)
    assert rc == -1


def test_amax_history_and_transpose_requantise(nv, native_lib):
    """MicroscaleManager.update_amax_history: history shifted by one, newest max |x| first (bf16 values, so the fp32
    maximum is exact), NaN ignored, unaligned and empty inputs; transpose_mxfp8: row-wise operand -> column-wise operand
    equals dequantise + column-wise quantise in the oracle."""
    from deepwell_b200 import cutlass_kernels as ck
    mm = ck.MicroscaleManager()
    hist = torch.tensor([3.0, 2.0, 1.0, 0.5], device="cuda")
    g = torch.Generator("cuda").manual_seed(77)
    x = (torch.randn(1000, 777, device="cuda", generator=g) * 3).bfloat16()
    x[5, 5] = float("nan")
    x[17, 100] = -123.5
    mm.update_amax_history(x, hist)
    assert hist.tolist() == [123.5, 3.0, 2.0, 1.0]
    mm.update_amax_history(x.flatten()[1:-1], hist)                 # 2-byte aligned view, tail path
    assert hist.tolist() == [123.5, 123.5, 3.0, 2.0]
    mm.update_amax_history(torch.empty(0, dtype=torch.bfloat16, device="cuda"), hist)
    assert hist.tolist() == [0.0, 123.5, 123.5, 3.0]
    big = torch.randn(4096, 4096, device="cuda", generator=g).bfloat16()
    mm.update_amax_history(big, hist)
    assert hist[0].item() == big.float().abs().max().item()
    assert native_lib.dw_mxfp8_update_amax_history(big.data_ptr(), None, 4, 16, None) == -1
    assert native_lib.dw_mxfp8_update_amax_history(big.data_ptr(), hist.data_ptr(), 0, 16, None) == -1
    # transpose with requantisation
    a = (torch.randn(256, 160, device="cuda", generator=g) * 2).bfloat16()
    codes, scales = mm.quantize_mxfp8(a)
    ct, st = mm.transpose_mxfp8(codes, scales)
    deq = o.f32_to_bf16_bits(o.dequantize_rowwise(codes.view(torch.uint8).cpu().numpy(), scales.cpu().numpy()))
    ec, es = o.quantize_colwise(deq)
    assert ct.shape == (160, 256) and np.array_equal(ct.view(torch.uint8).cpu().numpy(), ec)
    assert np.array_equal(st.cpu().numpy().reshape(es.shape), es)


@pytest.mark.parametrize("rule", [0, 1])
@pytest.mark.parametrize("layout_name", ["flat", "tiled"])
def test_rows_batch_is_the_single_quantisations_in_one_launch(nv, rule, layout_name):
    """dw_mxfp8_quantize_rows_batch: several matrices (here eleven, so two launches; sizes from one slab to several
    hundred, one empty) give byte for byte what dw_mxfp8_quantize gives for each, and one of them is checked against
    the C restatement."""
    layout = nv.SF_FLAT if layout_name == "flat" else nv.SF_TILED
    g = torch.Generator(device="cuda").manual_seed(99 + rule)
    shapes = [(128, 128), (4096, 4096), (1536, 4096), (1024, 14336), (256, 384), (0, 128), (2048, 1024), (128, 8192),
              (768, 4096), (512, 256), (3072, 768)]
    if layout == nv.SF_FLAT:
        shapes += [(100, 96), (33, 32)]                  # flat scales have no tile padding: any rows, cols % 32 == 0
    xs = []
    for r, k in shapes:
        x = torch.randn(r, k, device="cuda", generator=g) * 0.5
        if x.numel():
            x.view(-1)[:: 97] *= 40.0
        xs.append(x.bfloat16())
    codes = [torch.full((r, k), 0xEE, dtype=torch.uint8, device="cuda") for r, k in shapes]
    scales = [torch.full((nv.scale_bytes(r, k, layout),), 0xEE, dtype=torch.uint8, device="cuda") for r, k in shapes]
    launches = nv.quantize_rows_batch_into(xs, codes, scales, rule, layout)
    assert launches == -(-len(shapes) // nv.QUANT_BATCH_MAX)
    for x, gc, gs in zip(xs, codes, scales):
        if x.numel() == 0:
            continue
        ec, es = nv.quantize(x, nv.DIR_ROW, rule, layout)
        assert torch.equal(gc, ec.view(torch.uint8)) and torch.equal(gs, es.view(torch.uint8).reshape(-1))
    er, ers = c.quantize_rowwise(bits_of(xs[2]), rule)
    exp = ers if layout == nv.SF_FLAT else o.sf_flat_to_tiled(ers)
    assert np.array_equal(host(codes[2]), er) and np.array_equal(host(scales[2]), exp.reshape(-1))


def test_rows_batch_rejects_what_it_cannot_do(nv, native_lib):
    import ctypes
    x = torch.zeros(100, 128, dtype=torch.bfloat16, device="cuda")
    cbuf = torch.zeros(100, 128, dtype=torch.uint8, device="cuda")
    sbuf = torch.zeros(nv.scale_bytes(100, 128, nv.SF_TILED), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):                    # tiled scales with a ragged last row tile: no padding pass here
        nv.quantize_rows_batch_into([x], [cbuf], [sbuf], 0, nv.SF_TILED)
    n = nv.QUANT_BATCH_MAX + 1
    P, I = ctypes.c_void_p * n, ctypes.c_int64 * n
    rc = native_lib.dw_mxfp8_quantize_rows_batch(n, P(*[x.data_ptr()] * n), P(*[cbuf.data_ptr()] * n), P(*[sbuf.data_ptr()] * n),
                                                 I(*[100] * n), I(*[128] * n), 0, nv.SF_FLAT, 0, None)
    assert rc == -1                                      # DW_ERR_BAD_ARG: more matrices than one launch takes
    assert native_lib.dw_mxfp8_quantize_rows_batch(0, None, None, None, None, None, 0, nv.SF_FLAT, 0, None) == 0
