"""The reference's older linear-replacement API, rerouted to the MXFP8 path.

``optimize_for_blackwell`` -> ``optimize_model_inplace`` -> ``OptimizedLinear`` is the only route by
which the reference reaches a GEMM today (src/deepwell/__init__.py:191-223,
src/deepwell/kernels/production_kernels.py:353-408, :145-194); there the "MXFP8" precision ends in a
bf16 cuBLAS call and has no backward.  Here the same names give DWLinear, i.e. quantise +
block-scaled GEMM with autograd.  Only the linear pieces of that file exist (its attention and
benchmark helpers belong to another path).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import cutlass_kernels as _ext
from ..linear import DWLinear


@dataclass
class KernelConfig:
    """src/deepwell/kernels/production_kernels.py:19-27."""
    use_cutlass: bool = True
    use_tensor_cores: bool = True
    precision: str = "mxfp8"
    block_size: int = 32
    min_size_for_cutlass: int = 512
    batch_kernels: bool = True


class ProductionKernelManager:
    """gemm(a[M,K], b[K,N], bias) on the native kernels (reference :29-123).  The reference skips
    its kernel below 512^3 multiply-adds and falls back to torch; this one has no fallback."""

    def __init__(self, config: Optional[KernelConfig] = None):
        self.config = config or KernelConfig()
        self.cutlass_available = True
        self.cutlass_module = _ext

    def gemm(self, a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
             activation: Optional[str] = None) -> torch.Tensor:
        if not a.is_cuda:
            raise RuntimeError("ProductionKernelManager.gemm needs CUDA tensors")
        if self.config.precision == "mxfp8":
            out = _ext.mxfp8_gemm_bf16(a, b, bias=None if bias is None else bias.to(torch.bfloat16).contiguous())
        else:
            out = torch.matmul(a, b)
            if bias is not None:
                out = out + bias
        if activation == "relu":
            out = torch.relu(out)
        elif activation == "gelu":
            out = torch.nn.functional.gelu(out)
        return out if out.dtype == a.dtype else out.to(a.dtype)


class OptimizedLinear(DWLinear):
    """nn.Linear replacement of the reference (:145-194); same constructor, MXFP8 forward and backward."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 kernel_manager: Optional[ProductionKernelManager] = None):
        super().__init__(in_features, out_features, bias=bias)
        self.kernel_manager = kernel_manager or ProductionKernelManager()


def optimize_model_inplace(model: nn.Module, config: Optional[KernelConfig] = None) -> nn.Module:
    """Replaces every nn.Linear (features multiples of 32) in place, sharing its parameters (reference :353-408)."""
    config = config or KernelConfig()
    if config.precision != "mxfp8":
        return model
    from ..optimizer import DeepwellOptimizer
    DeepwellOptimizer(precision="mxfp8", verbose=False).optimize(model, inplace=True)
    return model


def optimize_for_blackwell(model: nn.Module, precision: str = "mxfp8", seq_len: int = 2048, batch_size: int = 32) -> nn.Module:
    """One-shot entry of the reference (src/deepwell/__init__.py:191-223): deep copy, then in-place replacement."""
    return optimize_model_inplace(copy.deepcopy(model), KernelConfig(precision=precision))
