"""GPU tests of the reference-facing layer: DWLinear / optimize() / the cutlass_kernels API."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import mx_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dw(native_lib):
    import deepwell_b200
    assert torch.cuda.is_available()
    return deepwell_b200


def bits_of(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def oracle_linear(x, w, b=None):
    y = o.bf16_bits_to_f32(o.mxfp8_linear(bits_of(x), bits_of(w), bias_bits=None if b is None else bits_of(b)))
    return torch.from_numpy(y)


def oracle_linear_f32(x, w, b=None):
    """fp32 result of the dequantised product (+ bias) before the bf16 rounding."""
    xc, xs = o.quantize_rowwise(bits_of(x))
    wc, ws = o.quantize_rowwise(bits_of(w))
    y = torch.from_numpy(o.dequantize_rowwise(xc, xs)) @ torch.from_numpy(o.dequantize_rowwise(wc, ws)).t()
    return y if b is None else y + b.float().cpu()[None, :]


def close(got, ref, rtol=1e-2):
    got, ref = got.double().cpu(), ref.double().cpu()
    return bool(((got - ref).abs() <= rtol * torch.maximum(ref.abs(), ref.abs().mean())).all())


def test_dwlinear_forward_backward_against_oracle(dw):
    torch.manual_seed(0)
    lin = nn.Linear(256, 384, bias=True).cuda().bfloat16()
    m = dw.DWLinear.from_linear(lin)
    x = torch.randn(4, 60, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)   # 240 tokens: padded to 256 for wgrad
    y = m(x)
    assert y.shape == (4, 60, 384)
    assert close(y.reshape(-1, 384), oracle_linear(x.reshape(-1, 256), lin.weight, lin.bias))
    gy = torch.randn_like(y)
    y.backward(gy)
    gy2, x2 = gy.reshape(-1, 384), x.detach().reshape(-1, 256)
    # dgrad: dY row-wise along N, W column-wise along N
    dyc, dys = o.quantize_rowwise(bits_of(gy2))
    wc, ws = o.quantize_rowwise(bits_of(lin.weight.detach().t().contiguous()))
    ref_dx = o.bf16_bits_to_f32(o.gemm_dequantized(dyc, dys, wc, ws))
    assert close(x.grad.reshape(-1, 256), torch.from_numpy(ref_dx))
    # wgrad: both operands column-wise along M (zero rows pad M to a multiple of 32)
    pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, (-t.shape[0]) % 32))
    ac, asc = o.quantize_rowwise(bits_of(pad(gy2).t().contiguous()))
    bc, bsc = o.quantize_rowwise(bits_of(pad(x2).t().contiguous()))
    ref_dw = o.bf16_bits_to_f32(o.gemm_dequantized(ac, asc, bc, bsc))
    assert close(lin.weight.grad, torch.from_numpy(ref_dw))
    assert close(lin.bias.grad, gy2.float().sum(0), rtol=2e-2)


def test_weight_cache_follows_parameter_updates(dw):
    m = dw.DWLinear(64, 64, bias=False).cuda().bfloat16()
    x = torch.randn(32, 64, device="cuda", dtype=torch.bfloat16)
    y1 = m(x)
    key = m._wq_key
    assert m(x).equal(y1) and m._wq_key == key
    with torch.no_grad():
        m.weight.mul_(2.0)
    y2 = m(x)
    assert m._wq_key != key and torch.equal(y2.float(), 2 * y1.float())       # power-of-two scaling is exact in MX


def test_optimize_trains_close_to_bf16(dw):
    """An MLP trained for a few SGD steps through optimize(precision='mxfp8') tracks the bf16 model."""
    torch.manual_seed(1)
    ref = nn.Sequential(nn.Linear(128, 512), nn.GELU(), nn.Linear(512, 128)).cuda().bfloat16()
    opt_model = dw.optimize(ref, precision="mxfp8", verbose=False)
    assert sum(isinstance(mm, dw.DWLinear) for mm in opt_model.modules()) == 2
    x = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    t = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    losses = []
    for model in (ref, opt_model):
        sgd = torch.optim.SGD(model.parameters(), lr=1e-2)
        cur = []
        for _ in range(5):
            sgd.zero_grad()
            loss = (model(x).float() - t.float()).pow(2).mean()
            loss.backward()
            sgd.step()
            cur.append(loss.item())
        losses.append(cur)
    assert losses[1][-1] < losses[1][0]
    assert all(abs(a - b) <= 0.05 * abs(a) for a, b in zip(*losses)), losses


def test_extension_module_api(dw):
    ck = dw.cutlass_kernels
    k = ck.BlackwellGemmKernel()
    k.initialize(256, 320, 512, "mxfp8", True, 32)
    a = torch.randn(256, 512, device="cuda").bfloat16()
    w = (torch.randn(320, 512, device="cuda") * 0.05).bfloat16()
    ref = oracle_linear(a, w)
    assert close(k.gemm(a, w.t()), ref)                        # b as the transposed view of an [N, K] weight
    assert close(k.gemm(a, w.t().contiguous()), ref)           # b as a contiguous [K, N] matrix
    c = torch.randn(256, 320, device="cuda").bfloat16()
    assert close(k.gemm(a, w.t(), c, 0.5, 2.0), 0.5 * ref + 2.0 * c.float().cpu(), rtol=2e-2)
    with pytest.raises(RuntimeError):
        k.gemm(a[:, :64], w.t())
    mm = ck.MicroscaleManager()
    codes, scales = mm.quantize_mxfp8(a, 32)
    assert codes.dtype == torch.float8_e4m3fn and codes.shape == a.shape and scales.dtype == torch.uint8
    ec, es = o.quantize_rowwise(bits_of(a))
    assert np.array_equal(codes.view(torch.uint8).cpu().numpy(), ec) and np.array_equal(scales.cpu().numpy(), es)
    back = mm.dequantize_mxfp8(codes, scales)
    assert np.array_equal(bits_of(back), o.f32_to_bf16_bits(o.dequantize_rowwise(ec, es)))
    ct, st = mm.quantize_mxfp8(a, 32, direction="col", scale_layout="tcgen05")
    assert ct.shape == (512, 256) and st.numel() == o.sf_tiled_size(512, 8)
    kb = ck.BlackwellGemmKernel()
    kb.initialize(256, 320, 512, "bf16")
    assert close(kb.gemm(a, w.t()), a.float().cpu() @ w.float().cpu().t(), rtol=2e-2)
    prof = ck.profile_kernel(k, 2, 3)
    assert prof["runtime_ms"] > 0 and prof["tflops"] > 0
    from deepwell_b200.kernels import CutlassKernel, GroupedGEMMKernel
    kk = CutlassKernel()
    kk.initialize(256, 320, 512, "mxfp8")
    assert close(kk.gemm(a, w.t()), ref)
    gk = GroupedGEMMKernel(2, 512, 320)
    outs = gk.grouped_gemm([a, a[:128]], [w.t(), w.t()])
    assert close(outs[0], ref) and close(outs[1], ref[:128])


class _Block(nn.Module):
    """Pre-LN decoder block built from plain nn.Linear projections + scaled_dot_product_attention
    (the 12-layer pre-LN decoder of the end-to-end training workload, scaled down)."""

    def __init__(self, hidden, heads, ffn):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(hidden), nn.LayerNorm(hidden)
        self.qkv, self.proj = nn.Linear(hidden, 3 * hidden), nn.Linear(hidden, hidden)
        self.up, self.down = nn.Linear(hidden, ffn), nn.Linear(ffn, hidden)

    def forward(self, x):
        b, s, h = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.heads, h // self.heads).permute(2, 0, 3, 1, 4)
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, h))
        return x + self.down(torch.nn.functional.gelu(self.up(self.ln2(x))))


class _Decoder(nn.Module):
    def __init__(self, vocab=1024, hidden=256, heads=4, ffn=1024, layers=2):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        self.blocks = nn.ModuleList([_Block(hidden, heads, ffn) for _ in range(layers)])
        self.ln_f = nn.LayerNorm(hidden)
        self.head = nn.Linear(hidden, vocab, bias=False)

    def forward(self, ids):
        x = self.embed(ids)
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.ln_f(x))


def test_optimize_decoder_training_step_tracks_bf16(dw):
    """deepwell.optimize(model, precision='mxfp8') on a small pre-LN decoder: every nn.Linear becomes a
    DWLinear, a few training steps run, and the loss curve stays within 3 % of the bf16 model's."""
    torch.manual_seed(5678)
    ref = _Decoder().cuda().bfloat16()
    model = dw.optimize(ref, precision="mxfp8", verbose=False)
    n_lin = sum(isinstance(m, nn.Linear) for m in ref.modules())
    assert sum(isinstance(m, dw.DWLinear) for m in model.modules()) == n_lin == 9
    ids = torch.randint(0, 1024, (4, 128), device="cuda")
    curves = []
    for net in (ref, model):
        opt = torch.optim.AdamW(net.parameters(), lr=1e-3)
        cur = []
        for _ in range(6):
            opt.zero_grad()
            logits = net(ids)
            loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 1024).float(), ids[:, 1:].reshape(-1))
            loss.backward()
            opt.step()
            cur.append(loss.item())
        curves.append(cur)
    assert curves[1][-1] < curves[1][0] - 0.3, curves
    assert all(abs(a - b) <= 0.03 * abs(a) for a, b in zip(*curves)), curves


def test_dwlinear_training_step_captured_in_a_cuda_graph(dw):
    """Forward + backward of a DWLinear captured in a CUDA graph (all launches go to the capturing stream, outputs come
    from torch's allocator, nothing synchronises) and replayed on new input values: same gradients as the eager run."""
    torch.manual_seed(31)
    m = dw.DWLinear.from_linear(nn.Linear(256, 384, bias=True).cuda().bfloat16())
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)

    def step():
        x.grad = None
        m.weight.grad = None
        m.bias.grad = None
        y = m(x)
        y.backward(gy)
        return y

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    x.grad = None
    m.weight.grad = None
    m.bias.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = step()
    # new values in the captured input buffers
    with torch.no_grad():
        x.copy_(torch.randn(512, 256, device="cuda").bfloat16())
        gy.copy_(torch.randn(512, 384, device="cuda").bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    got = [y_static.clone(), x.grad.clone(), m.weight.grad.clone(), m.bias.grad.clone()]
    y = step()
    torch.cuda.synchronize()
    want = [y, x.grad, m.weight.grad, m.bias.grad]
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    from deepwell_b200 import _native
    _native.check_status()


def test_captured_graph_sees_weight_updates(dw):
    """A forward + backward captured in a CUDA graph re-quantises the weight on every replay, into the module's own
    persistent buffers: after the weight is changed through ``p.data.copy_`` (which moves no version counter), after a
    real optimizer step, and after eager forwards in between, a replay equals the eager run on the current weight."""
    torch.manual_seed(33)
    m = dw.DWLinear.from_linear(nn.Linear(256, 384, bias=True).cuda().bfloat16())
    opt = torch.optim.SGD(m.parameters(), lr=0.5)
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)

    def step():
        x.grad = None
        m.weight.grad = None
        m.bias.grad = None
        y = m(x)
        y.backward(gy)
        return y

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    x.grad = None
    m.weight.grad = None
    m.bias.grad = None
    buffers = [t.data_ptr() for pair in (m._wq_row, m._wq_col) for t in pair]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = step()
    assert [t.data_ptr() for pair in (m._wq_row, m._wq_col) for t in pair] == buffers      # never replaced
    static = [y_static, x.grad, m.weight.grad, m.bias.grad]       # the tensors every replay writes (an eager step rebinds .grad)

    def replay_equals_eager():
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in static]
        y = step()
        torch.cuda.synchronize()
        for a, b in zip(got, [y, x.grad, m.weight.grad, m.bias.grad]):
            assert torch.equal(a, b)
        return got[0]

    y0 = replay_equals_eager()
    new_w = (torch.randn(384, 256, device="cuda") * 0.1).bfloat16()
    version = m.weight._version
    m.weight.data.copy_(new_w)                               # master-weight style write: no version bump
    assert m.weight._version == version
    y1 = replay_equals_eager()                               # eager run inside also refreshes: see invalidate below
    assert not torch.equal(y0, y1)
    step()
    opt.step()                                               # in-place update under no_grad: version moves
    y2 = replay_equals_eager()
    assert not torch.equal(y1, y2)
    assert [t.data_ptr() for pair in (m._wq_row, m._wq_col) for t in pair] == buffers
    from deepwell_b200 import _native
    _native.check_status()


def test_data_writes_need_invalidate_or_cache_off(dw):
    """Outside graph capture the weight operands are refreshed when the parameter's version moves.  A write through
    ``weight.data`` moves no version: ``invalidate_weight_cache()`` (or ``weight_cache="off"``) makes it visible."""
    m = dw.DWLinear(64, 96, bias=False).cuda().bfloat16()
    x = torch.randn(32, 64, device="cuda", dtype=torch.bfloat16)
    y1 = m(x)
    m.weight.data.mul_(2.0)
    m.invalidate_weight_cache()
    assert torch.equal(m(x).float(), 2 * y1.float())
    off = dw.DWLinear(64, 96, bias=False, weight_cache="off").cuda().bfloat16()
    z1 = off(x)
    off.weight.data.mul_(2.0)                                # no invalidate needed
    assert torch.equal(off(x).float(), 2 * z1.float())


def test_grouped_weight_cache_never_matches_recycled_temporaries(dw):
    """Weight lists rebuilt from temporaries on every call (fresh tensors, version 0, addresses the allocator may
    hand out again) must not hit an entry built from other values: the entry keeps its sources alive and is matched by
    storage identity, not by address."""
    from deepwell_b200 import cutlass_kernels as ck
    K, N, G = 256, 256, 2
    g = torch.Generator("cpu").manual_seed(5)
    a_list = [torch.randn(256, K, generator=g).bfloat16().cuda() for _ in range(G)]
    masters = [(torch.randn(N, K, generator=g) * 0.05).cuda() for _ in range(G)]           # fp32 master weights
    cache = {}
    outs = []
    for scale in (1.0, 2.0, 4.0):
        w_list = [(w * scale).to(torch.bfloat16).t() for w in masters]                      # temporaries, rebuilt each call
        outs.append([o_.clone() for o_ in ck.mxfp8_grouped_gemm_bf16(a_list, w_list, weight_cache=cache)])
        del w_list
    for o1, o2, o4 in zip(*outs):
        assert torch.equal(o2.float(), 2 * o1.float()) and torch.equal(o4.float(), 4 * o1.float())   # exact in MX
    # unchanged persistent weights do hit
    w_keep = [(w).to(torch.bfloat16).t() for w in masters]
    ck.mxfp8_grouped_gemm_bf16(a_list, w_keep, weight_cache=cache)
    operand = cache["operand"][0]
    ck.mxfp8_grouped_gemm_bf16(a_list, [w for w in w_keep], weight_cache=cache)
    assert cache["operand"][0] is operand


def test_blackwell_production_gemm_and_fused_linear_gelu(dw):
    """deepwell.kernels.blackwell_production: BlackwellGEMM.gemm with bias + activation fused in the epilogue equals the
    oracle's activation of the fp32 result (tolerance 1e-2 of the value scale, bf16 output); FusedLinearGELU without
    autograd equals that, with autograd equals DWLinear + F.gelu and trains; BlackwellGroupedGEMM splits like a loop."""
    from deepwell_b200.kernels.blackwell_production import (BlackwellConfig, BlackwellGEMM, BlackwellGroupedGEMM,
                                                            FusedLayerNormLinear, FusedLinearGELU,
                                                            optimize_model_for_blackwell)
    torch.manual_seed(41)
    x = torch.randn(300, 256, device="cuda").bfloat16()
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16()
    b = torch.randn(384, device="cuda").bfloat16()
    pre = torch.from_numpy(o.bf16_bits_to_f32(o.mxfp8_linear(bits_of(x), bits_of(w), bias_bits=bits_of(b)))).float()
    exact = oracle_linear_f32(x, w, b)
    g = BlackwellGEMM(BlackwellConfig())
    assert close(g.gemm(x, w.t(), bias=b), pre)
    for act, fn in (("gelu", torch.nn.functional.gelu), ("relu", torch.relu), ("silu", torch.nn.functional.silu)):
        assert close(g.gemm(x, w.t(), bias=b, activation=act), fn(exact), rtol=1e-2)
    unfused = BlackwellGEMM(BlackwellConfig(fuse_gelu=False, fuse_bias=False))
    assert close(unfused.gemm(x, w.t(), bias=b, activation="gelu"), torch.nn.functional.gelu(exact), rtol=2e-2)
    layer = FusedLinearGELU(256, 384).cuda()
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.bias.copy_(b)
        y_inf = layer(x.view(3, 100, 256))
    assert y_inf.shape == (3, 100, 384) and close(y_inf.reshape(-1, 384), torch.nn.functional.gelu(exact), rtol=1e-2)
    xg = x.clone().requires_grad_(True)
    y_train = layer(xg)
    y_train.float().square().mean().backward()
    assert close(y_train, torch.nn.functional.gelu(pre), rtol=1e-2)
    assert xg.grad is not None and layer.weight.grad is not None and layer.bias.grad is not None
    outs = BlackwellGroupedGEMM().grouped_gemm([x, x[:77]], [w.t(), w.t()])
    assert close(outs[0], g.gemm(x, w.t())) and outs[1].shape == (77, 384)
    ln = FusedLayerNormLinear(256, 128).cuda()
    assert ln(x).shape == (300, 128)
    seq = optimize_model_for_blackwell(nn.Sequential(nn.Linear(256, 128), nn.GELU(), nn.Linear(128, 64)).cuda().bfloat16())
    assert isinstance(seq[0], dw.DWLinear) and isinstance(seq[2], dw.DWLinear)


def test_fused_swiglu_mlp_equals_the_unfused_layers(dw):
    """FusedSwiGLUMLP without autograd (gate+up GEMM with the gated epilogue writing the down projection's operand) gives
    the bits of the three separate MXFP8 layers whenever those round the same way, i.e. within the GEMM tolerance of
    them always; with autograd it IS the three layers and trains."""
    from deepwell_b200.kernels.blackwell_production import FusedSwiGLUMLP
    torch.manual_seed(7)
    m = FusedSwiGLUMLP(256, 704).cuda()               # F = 704 = 5.5 scale tiles: padded k-blocks on the output
    x = torch.randn(3, 100, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        y_fused = m(x)
        m.fuse = False
        y_three = m(x)
        m.fuse = True
    assert y_fused.shape == (3, 100, 256)
    # the unfused path rounds gate and up to bf16 before the product and the fused one keeps them in fp32, so a few E4M3
    # codes of the hidden activation differ by one step: compared in the Frobenius norm, not element by element
    assert ((y_fused.float() - y_three.float()).norm() / y_three.float().norm()).item() < 2e-2
    ref = torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(x.float(), m.gate_proj.weight.float()))
                                     * torch.nn.functional.linear(x.float(), m.up_proj.weight.float()), m.down_proj.weight.float())
    assert ((y_fused.float() - ref).norm() / ref.norm()).item() < 0.15        # five E4M3 roundings (x, gate, up, h, down) against fp32
    xg = x.clone().requires_grad_(True)
    m(xg).float().pow(2).mean().backward()
    assert xg.grad is not None and m.gate_proj.weight.grad is not None and m.down_proj.weight.grad is not None
    with torch.no_grad():                              # a weight update reaches the cached interleaved operand
        m.gate_proj.weight.mul_(2.0)
        y2 = m(x)
    assert not torch.equal(y2, y_fused)
    from deepwell_b200 import _native
    _native.check_status()


def test_engine_mlp_executor(dw):
    """ExecutableModel._mlp_with_cutlass (the reference's second caller of the GEMM, src/deepwell/engine.py:132-209):
    Linear -> GELU -> Linear runs as two GEMMs with the fused epilogue and equals FusedMLP's bits; a lone Linear with a
    ReLU, layers the path does not cover (LayerNorm, a Linear with odd features) and a 3-D input are handled."""
    import deepwell
    from deepwell.engine import ExecutableModel
    from deepwell_b200.kernels.blackwell_production import FusedMLP
    torch.manual_seed(3)
    fm = FusedMLP(128, 512, activation="gelu").cuda()
    mlp = nn.Sequential(nn.Linear(128, 512), nn.GELU(), nn.Linear(512, 128)).cuda().bfloat16()
    with torch.no_grad():
        mlp[0].weight.copy_(fm.up.weight); mlp[0].bias.copy_(fm.up.bias)
        mlp[2].weight.copy_(fm.down.weight); mlp[2].bias.copy_(fm.down.bias)
    ex = ExecutableModel(None, mlp)
    x = torch.randn(4, 40, 128, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = fm(x)
    got = ex._mlp_with_cutlass(x, mlp, 0)
    assert got.shape == (4, 40, 128) and torch.equal(got, want)
    assert torch.equal(ex._mlp_with_cutlass(x, mlp, 0), want)                 # cached weight operands
    with torch.no_grad():
        mlp[0].weight.mul_(2.0)
    assert not torch.equal(ex._mlp_with_cutlass(x, mlp, 0), want)             # ... follow the parameter
    odd = nn.Sequential(nn.LayerNorm(128), nn.Linear(128, 96), nn.ReLU(), nn.Linear(96, 50)).cuda().bfloat16()
    got = ex._mlp_with_cutlass(x, odd, 1)
    with torch.no_grad():
        ref = odd(x)
    assert got.shape == ref.shape
    assert ((got.float() - ref.float()).norm() / ref.float().norm()).item() < 0.06
    assert torch.equal(ex(x), mlp(x))                                          # forward runs the original model
    from deepwell_b200 import _native
    _native.check_status()


def test_fused_mlp_inference_equals_the_unfused_layers(dw):
    """FusedMLP without autograd (hidden activation quantised in the first GEMM's epilogue, never written in bf16)
    against the same module with autograd enabled (DWLinear, torch GELU on the bf16 result, DWLinear): the fused path
    applies the activation to the fp32 accumulator, so the hidden values differ by one bf16 rounding before they are
    quantised; where that moves an E4M3 code (steps of 6-12 %) one term of the second contraction changes, so the
    outputs are compared in norm: relative Frobenius error <= 3e-2 (the bit-level check of the fused epilogue is in
    test_gpu_gemm.py); the fused path is deterministic."""
    from deepwell_b200.kernels.blackwell_production import FusedMLP
    torch.manual_seed(43)
    mlp = FusedMLP(256, 1024, 256, activation="gelu").cuda()
    x = torch.randn(4, 96, 256, device="cuda").bfloat16()
    with torch.no_grad():
        y1 = mlp(x)
        y2 = mlp(x)
    assert y1.shape == (4, 96, 256) and torch.equal(y1, y2)
    y_ref = mlp(x)                       # parameters require grad: the unfused path
    assert y_ref.requires_grad
    err = (y1.float() - y_ref.detach().float()).norm() / y_ref.detach().float().norm()
    assert err.item() <= 3e-2, err.item()
    y_ref.float().square().mean().backward()
    assert mlp.up.weight.grad is not None and mlp.down.weight.grad is not None
    from deepwell_b200 import _native
    _native.check_status()
