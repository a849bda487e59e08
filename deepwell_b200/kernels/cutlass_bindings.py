"""Python kernel API — drop-in for the reference's ``deepwell.kernels.cutlass_bindings``.

Public names follow src/deepwell/kernels/cutlass_bindings.py of the reference: availability
flags (:17-49), CutlassConfig (:73-91), CutlassKernel (:94-361), GroupedGEMMKernel (:364-480),
BlackwellMMATensor (:483-577).  Behavioural changes:

  * ``precision="mxfp8"`` reaches the MXFP8 kernel.  The reference maps "mxfp8" to
    torch.bfloat16 and then to the dtype string "bf16" (:336, :350-361), so its native MXFP8
    branch can never be selected through this wrapper;
  * there is one backend, the native library of this package: no pycutlass path, no PyTorch
    fallback (:188-192, :294-298).  CPU tensors raise RuntimeError.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import _native as nv
from .. import cutlass_kernels as _cutlass_ext

# The CUTLASS Python builder API is not a dependency of this package.
CUTLASS_PYTHON_AVAILABLE = False
try:
    nv.load()
    CUTLASS_CPP_AVAILABLE = True
except nv.NativeLibraryError:           # the library must be built; callers see a clear error on use
    CUTLASS_CPP_AVAILABLE = False
CUTLASS_AVAILABLE = CUTLASS_CPP_AVAILABLE

_PRECISION_TO_EXT = {"fp32": "fp32", "fp16": "fp16", "bf16": "bf16", "bfloat16": "bf16", "mxfp8": "mxfp8"}
_TORCH_TO_EXT = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}


@dataclass
class CutlassConfig:
    """Tile configuration.  Defaults describe the kernel this package launches: a 128 x 256
    accumulator tile per CTA, 128 bytes of K per pipeline stage, tcgen05 MMA shape 128x256x32."""
    tile_m: int = 128
    tile_n: int = 256
    tile_k: int = 128
    stages: int = 4
    warp_count: Tuple[int, int, int] = (6, 1, 1)          # producer, MMA issuer, four epilogue warps
    instruction_shape: Tuple[int, int, int] = (128, 256, 32)
    cluster_shape: Tuple[int, int, int] = (1, 1, 1)
    epilogue_functor: str = "LinearCombination"
    swizzle: int = 1
    use_tcgen05: bool = True
    tmem_residency: bool = True
    microscale_block_size: int = 32
    force_tcgen05: bool = True


def _require_native() -> None:
    if not CUTLASS_AVAILABLE:
        nv.load()       # raises NativeLibraryError with build instructions


class CutlassKernel:
    """GEMM front-end with a per-problem cache of native kernel objects."""

    def __init__(self, config: Optional[CutlassConfig] = None):
        self.config = config or CutlassConfig()
        self.kernel_cache: Dict[str, Any] = {}
        self.is_initialized = False
        self.current_kernel = None
        self.precision = "bf16"

    def _get_kernel_key(self, m: int, n: int, k: int, dtype_a: str, dtype_b: str, dtype_c: str) -> str:
        return f"{m}x{n}x{k}_{dtype_a}_{dtype_b}_{dtype_c}"

    def _native_kernel(self, m: int, n: int, k: int, ext_dtype: str, use_microscaling: bool, block_size: int):
        key = self._get_kernel_key(m, n, k, ext_dtype, ext_dtype, ext_dtype)
        kernel = self.kernel_cache.get(key)
        if kernel is None:
            kernel = _cutlass_ext.BlackwellGemmKernel()
            kernel.initialize(m, n, k, ext_dtype, use_microscaling, block_size)
            if self.config.use_tcgen05:
                kernel.enable_tmem_residency(self.config.tmem_residency)
            self.kernel_cache[key] = kernel
        return kernel

    def initialize(self, m: int = None, n: int = None, k: int = None, precision: str = "bf16",
                   use_microscaling: bool = False, block_size: int = 32):
        if m is None or n is None or k is None:     # legacy no-argument form
            self.is_initialized = True
            return
        _require_native()
        self.m, self.n, self.k = m, n, k
        self.precision, self.use_microscaling, self.block_size = precision, use_microscaling, block_size
        ext = _PRECISION_TO_EXT.get(precision)
        if ext is None:
            raise RuntimeError(f"precision {precision!r} has no kernel in this package")
        self.current_kernel = self._native_kernel(m, n, k, ext, use_microscaling or ext == "mxfp8", block_size)
        self.is_initialized = True

    def gemm(self, a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0,
             beta: float = 0.0, use_microscaling: bool = True) -> torch.Tensor:
        """alpha * a[M,K] @ b[K,N] + beta * c on the native kernels."""
        _require_native()
        if not a.is_cuda or not b.is_cuda:
            raise RuntimeError("CutlassKernel.gemm needs CUDA tensors; this package has no CPU path")
        m, k = a.shape
        n = b.shape[1]
        ext = "mxfp8" if self.precision == "mxfp8" else _TORCH_TO_EXT.get(a.dtype, "bf16")
        kernel = self._native_kernel(m, n, k, ext, use_microscaling and ext == "mxfp8", self.config.microscale_block_size)
        return kernel.gemm(a, b, c, alpha, beta)

    # kept for callers that used the reference's private helpers
    def _gemm_cutlass_cpp(self, a, b, c, alpha, beta):
        return self.gemm(a, b, c, alpha, beta)

    def _dtype_to_cutlass_str(self, dtype: torch.dtype) -> str:
        return {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16", torch.int8: "int8"}.get(dtype, "fp16")

    def _precision_to_dtype(self, precision: str) -> torch.dtype:
        """Storage dtype of the operands handed to gemm() for a precision string."""
        return {"fp32": torch.float32, "fp16": torch.float16, "int8": torch.int8}.get(precision, torch.bfloat16)


class GroupedGEMMKernel(CutlassKernel):
    """One GEMM per expert on the same kernel (src/deepwell/kernels/cutlass_bindings.py:364-480)."""

    def __init__(self, num_experts: int, expert_dim: int, hidden_dim: int, config: Optional[CutlassConfig] = None):
        super().__init__(config)
        self.num_experts, self.expert_dim, self.hidden_dim = num_experts, expert_dim, hidden_dim

    def grouped_gemm(self, inputs: List[torch.Tensor], weights: List[torch.Tensor],
                     biases: Optional[List[torch.Tensor]] = None, activation: str = "none") -> List[torch.Tensor]:
        if len(inputs) != self.num_experts:
            raise ValueError(f"Expected {self.num_experts} inputs, got {len(inputs)}")
        if len(weights) != self.num_experts:
            raise ValueError(f"Expected {self.num_experts} weights, got {len(weights)}")
        _require_native()
        kernel = self.kernel_cache.get("grouped_gemm")
        if kernel is None or isinstance(kernel, dict):
            kernel = _cutlass_ext.BlackwellGroupedGemmKernel()
            sizes = [(x.shape[0], w.shape[1], x.shape[1]) for x, w in zip(inputs, weights)]
            mx = bool(self.config and self.config.use_tcgen05)
            kernel.initialize(sizes, "mxfp8" if mx else "bf16", mx)
            kernel.set_expert_parallel_strategy(True)
            self.kernel_cache["grouped_gemm"] = kernel
        outputs = kernel.grouped_gemm(inputs, weights)
        if biases is not None:
            outputs = [o + b for o, b in zip(outputs, biases)]
        if activation == "relu":
            outputs = [torch.relu(o) for o in outputs]
        elif activation == "gelu":
            outputs = [torch.nn.functional.gelu(o) for o in outputs]
        return outputs

    def build_grouped_kernel(self, batch_sizes: List[int], dtype: str = "mxfp8"):
        self.kernel_cache["grouped_gemm"] = {
            "num_groups": self.num_experts, "batch_sizes": batch_sizes, "expert_dim": self.expert_dim,
            "hidden_dim": self.hidden_dim, "dtype": dtype, "use_microscaling": dtype in ("mxfp8", "nvfp4"),
            "sm_version": 100,
        }


class BlackwellMMATensor:
    """Static facts about the tcgen05 path (src/deepwell/kernels/cutlass_bindings.py:483-577)."""

    # nominal dense B200 peaks, TFLOP/s
    _PEAK = {"nvfp4": 9000.0, "mxfp4": 9000.0, "mxfp8": 4500.0, "fp8": 4500.0}

    def __init__(self):
        self.sm_version = 100
        self.supports_mxfp8 = True
        self.supports_nvfp4 = False       # no FP4 kernel in this package
        self.tmem_size_kb = 256

    def can_use_tmem_residency(self, accumulator_size_bytes: int) -> bool:
        """A CTA owns 128 lanes x 512 columns x 4 bytes of tensor memory."""
        return accumulator_size_bytes <= self.tmem_size_kb * 1024

    def get_optimal_tile_size(self, m: int, n: int, k: int, dtype: str) -> Tuple[int, int, int]:
        if dtype in ("mxfp8", "fp8"):
            return (128, 256, 128) if n > 128 else (128, 128, 128)
        if dtype in ("nvfp4", "mxfp4"):
            return (128, 256, 256)
        return (128, 256, 64)

    def estimate_performance(self, m: int, n: int, k: int, dtype: str) -> Dict[str, float]:
        peak = self._PEAK.get(dtype, 2250.0)
        flops = 2 * m * n * k
        work = m * n * k
        efficiency = 0.3 if work < 1e6 else (0.7 if work < 1e9 else 0.9)
        achieved = peak * efficiency
        return {"flops": flops, "peak_tflops": peak, "achieved_tflops": achieved, "efficiency": efficiency,
                "time_ms": (flops / 1e12) / achieved * 1000}


def build_cutlass_extension():
    """Builds the native library in-tree (the reference's function only warned, :580-592)."""
    from .. import _build
    return _build.build()
