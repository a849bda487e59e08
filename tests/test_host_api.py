"""CPU tests of the host-side mirror of the reference interface (registry, optimizer, wrappers)."""
import pytest
import torch
import torch.nn as nn


def test_registry_semantics(native_lib):
    from deepwell_b200.kernels.registry import KernelBackend, KernelRegistry, KernelSpec, get_registry, register_kernel
    r = get_registry()
    k = r.find_kernel("gemm", "mxfp8", 100)
    assert k.name == "cutlass_sm100_mxfp8_gemm" and k.has_microscaling and (128, 256, 128) in k.tile_sizes
    assert r.find_kernel("gemm", "mxfp8", 90) is None                      # needs Blackwell
    assert r.find_kernel("gemm", "fp8", 90).name == "cutlass_sm90_fp8_gemm"
    assert r.find_kernel("gemm", "bf16", 100).name == "cublas_gemm"
    assert r.find_kernel("attention", "bf16", 100).name == "te_attention"
    assert r.find_kernel("nosuch", "bf16", 100) is None
    assert r.find_kernel("quantize", "mxfp8", 100).name == "sm100_mxfp8_quantize"
    chain = [s.name for s in r.find_fallback_chain("gemm", "mxfp8", 100)]
    assert chain == ["cutlass_sm100_mxfp8_gemm", "cutlass_sm90_fp8_gemm", "cublas_gemm", "torch_linear"]
    assert r.get_kernel_info("te_mxfp8_linear").backend is KernelBackend.TE
    assert "cutlass_sm100_mxfp8_gemm" not in r.validate_for_hardware(90)["gemm"]
    assert len(r.list_kernels()) >= 10 and len(r.list_kernels("gemm")) == 4
    fresh = KernelRegistry()
    fresh.register(KernelSpec("mine", KernelBackend.CUSTOM, "gemm", 100, ["MXFP8"], has_microscaling=True, is_fused=True))
    # same fused/microscaling flags but CUSTOM backend scores below CUTLASS
    assert fresh.find_kernel("gemm", "mxfp8", 100).name == "cutlass_sm100_mxfp8_gemm"
    assert fresh.find_kernel("gemm", "mxfp8", 100, require_microscaling=True).supports_precision("mxfp8")
    register_kernel(KernelSpec("tmp_op", KernelBackend.TORCH, "tmp", 0, ["fp32"]))
    assert get_registry().find_kernel("tmp", "fp32", 0).name == "tmp_op"


def test_optimize_replaces_linears(native_lib, capsys):
    import deepwell_b200 as dw

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1 = nn.Linear(64, 128)
            self.act = nn.GELU()
            self.fc2 = nn.Linear(128, 64, bias=False)
            self.head = nn.Linear(64, 10)          # 10 is not a multiple of 32 -> kept

        def forward(self, x):
            return self.head(self.fc2(self.act(self.fc1(x))))

    model = nn.Sequential(Block(), Block())
    opt = dw.DeepwellOptimizer(precision="mxfp8", verbose=True)
    new = opt.optimize(model)
    out = capsys.readouterr().out
    assert "[0.fc1] Linear -> DWLinear" in out and "Total modules replaced: 4" in out
    assert opt.stats == {"modules_replaced": 4, "attention_modules": 0, "linear_modules": 4, "other_modules": 0}
    assert isinstance(new[0].fc1, dw.DWLinear) and isinstance(new[1].fc2, dw.DWLinear)
    assert type(new[0].head) is nn.Linear and len(opt.skipped) == 2
    assert type(model[0].fc1) is nn.Linear                                   # deep copy: original untouched
    assert new.state_dict().keys() == model.state_dict().keys()              # checkpoints interchange
    assert torch.equal(new[0].fc1.weight, model[0].fc1.weight) and new[0].fc1.weight is not model[0].fc1.weight
    same = dw.optimize(model, precision="mxfp8", verbose=False, inplace=True)
    assert same is model and isinstance(model[0].fc1, dw.DWLinear)
    untouched = dw.optimize(nn.Sequential(nn.Linear(64, 64)), precision="bf16", verbose=False)
    assert type(untouched[0]) is nn.Linear                                   # only mxfp8 rewrites Linear
    with pytest.raises(RuntimeError):
        new[0].fc1(torch.randn(4, 64))                                       # no CPU path
    with pytest.raises(ValueError):
        dw.DWLinear(30, 64)


def test_wrappers_refuse_cpu_tensors(native_lib):
    from deepwell_b200 import cutlass_kernels as ck
    from deepwell_b200.kernels import cutlass_bindings as cb
    assert cb.CUTLASS_AVAILABLE and cb.CUTLASS_CPP_AVAILABLE and not cb.CUTLASS_PYTHON_AVAILABLE
    assert ck.CUTLASS_PYTHON_FALLBACK is False
    k = ck.BlackwellGemmKernel()
    k.initialize(128, 128, 128, "mxfp8", True, 32)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        k.gemm(torch.randn(128, 128), torch.randn(128, 128))
    with pytest.raises(RuntimeError):
        k.initialize(128, 128, 128, "nvfp4")
    with pytest.raises(RuntimeError):
        ck.MicroscaleManager().quantize_mxfp8(torch.randn(4, 32))
    assert k.get_expected_tflops() == 4500.0 * 0.5
    kk = cb.CutlassKernel()
    kk.initialize()
    assert kk.is_initialized
    kk.initialize(256, 256, 256, "mxfp8")
    assert kk.current_kernel.dtype == "mxfp8"                                # "mxfp8" reaches the MXFP8 kernel
    with pytest.raises(RuntimeError):
        kk.gemm(torch.randn(4, 4), torch.randn(4, 4))
    assert ck.PrecisionType.MXFP8.name == "MXFP8" and len(ck.PrecisionType) == 10
    t = cb.BlackwellMMATensor()
    assert t.get_optimal_tile_size(4096, 4096, 4096, "mxfp8") == (128, 256, 128)
    assert t.can_use_tmem_residency(128 * 256 * 4)


def test_shard_bounds():
    from deepwell_b200.sharded import shard_bounds
    for n, w in [(4096, 8), (6144, 8), (28672, 8), (4096, 3), (96, 4)]:
        spans = [shard_bounds(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((b - a) % 32 == 0 for a, b in spans)
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 32
    assert shard_bounds(28672, 8, 3) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        shard_bounds(100, 2, 0)


def test_reference_import_names(native_lib):
    """Code written against the reference package imports unchanged."""
    import deepwell
    from deepwell import cutlass_kernels
    from deepwell.kernels import CutlassKernel, get_registry
    from deepwell.kernels.cutlass_bindings import CUTLASS_AVAILABLE
    from deepwell.kernels.registry import KernelSpec
    from deepwell.optimizer import DeepwellOptimizer
    import deepwell_b200
    assert deepwell.optimize is deepwell_b200.optimize and CUTLASS_AVAILABLE
    assert cutlass_kernels.BlackwellGemmKernel is deepwell_b200.cutlass_kernels.BlackwellGemmKernel
    assert get_registry().find_kernel("gemm", "mxfp8", 100).name == "cutlass_sm100_mxfp8_gemm"
    assert KernelSpec and CutlassKernel and DeepwellOptimizer


def test_legacy_linear_replacement_names(native_lib):
    """optimize_for_blackwell / optimize_model_inplace / OptimizedLinear of the reference lead to DWLinear."""
    import deepwell
    from deepwell.kernels.production_kernels import KernelConfig, OptimizedLinear, ProductionKernelManager, optimize_model_inplace
    import deepwell_b200 as dw
    model = nn.Sequential(nn.Embedding(100, 64), nn.LayerNorm(64), nn.Linear(64, 96))
    new = deepwell.optimize_for_blackwell(model, precision="mxfp8", seq_len=8, batch_size=2)
    assert isinstance(new[2], dw.DWLinear) and type(model[2]) is nn.Linear
    same = optimize_model_inplace(model, KernelConfig(precision="mxfp8"))
    assert same is model and isinstance(model[2], dw.DWLinear)
    lin = OptimizedLinear(64, 32, bias=False)
    assert isinstance(lin, dw.DWLinear) and lin.bias is None and isinstance(lin.kernel_manager, ProductionKernelManager)
    with pytest.raises(RuntimeError):
        ProductionKernelManager().gemm(torch.randn(4, 32), torch.randn(32, 32))


def test_optimize_honours_a_precision_policy(native_lib):
    """Layers a precision policy names sensitive stay unreplaced: by substring list, or by an object shaped like the
    reference's PrecisionPolicy (policy.config.sensitive_layers, src/deepwell/precision/policy.py:102-109)."""
    import types
    import deepwell_b200 as dw

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.first_linear = nn.Linear(64, 64)
            self.body = nn.Sequential(nn.Linear(64, 128), nn.Linear(128, 64))
            self.logits = nn.Linear(64, 96)

    opt = dw.DeepwellOptimizer(precision="mxfp8", verbose=False, sensitive_layers=["logits", "First_Linear"])
    new = opt.optimize(Net())
    assert type(new.first_linear) is nn.Linear and type(new.logits) is nn.Linear
    assert isinstance(new.body[0], dw.DWLinear) and isinstance(new.body[1], dw.DWLinear)
    assert opt.stats["linear_modules"] == 2 and {n for n, _ in opt.skipped} == {"first_linear", "logits"}
    policy = types.SimpleNamespace(config=types.SimpleNamespace(sensitive_layers=["embedding", "logits"]))
    new = dw.optimize(Net(), precision="mxfp8", verbose=False, policy=policy)
    assert type(new.logits) is nn.Linear and isinstance(new.first_linear, dw.DWLinear)
    everything = dw.optimize(Net(), precision="mxfp8", verbose=False)
    assert sum(isinstance(m, dw.DWLinear) for m in everything.modules()) == 4
