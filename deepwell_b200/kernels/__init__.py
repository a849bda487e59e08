"""Kernel-facing API (registry + GEMM front-end), mirroring ``deepwell.kernels`` of the reference
(src/deepwell/kernels/__init__.py:5-34) for the MXFP8 linear path."""
from .registry import KernelBackend, KernelRegistry, KernelSpec, get_registry, register_kernel
from .cutlass_bindings import (CUTLASS_AVAILABLE, BlackwellMMATensor, CutlassConfig, CutlassKernel,
                               GroupedGEMMKernel)

__all__ = ["KernelBackend", "KernelRegistry", "KernelSpec", "get_registry", "register_kernel", "CUTLASS_AVAILABLE",
           "BlackwellMMATensor", "CutlassConfig", "CutlassKernel", "GroupedGEMMKernel"]
