"""Kernel registry — the lookup API of the reference's ``deepwell.kernels.registry``.

Same public names and selection semantics as src/deepwell/kernels/registry.py:9-328 of the
reference (KernelBackend, KernelSpec, KernelRegistry.{register, find_kernel,
find_fallback_chain, get_kernel_info, list_kernels, validate_for_hardware}, get_registry,
register_kernel).  The default table keeps the reference's entries (names included, tests of
the reference print them, tests/test_basic_api.py:170-183) with two changes: the tile sizes of
``cutlass_sm100_mxfp8_gemm`` are the ones the tcgen05 kernel of this package really uses, and a
``quantize`` entry describes the MX quantiser.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Dict, List, Optional, Tuple


class KernelBackend(enum.Enum):
    CUTLASS = "cutlass"
    TE = "transformer_engine"
    CUBLAS = "cublas"
    TRITON = "triton"
    TORCH = "torch"
    CUSTOM = "custom"


@dataclasses.dataclass
class KernelSpec:
    name: str
    backend: KernelBackend
    op_type: str
    sm_version: int
    precision_support: List[str]
    has_microscaling: bool = False
    is_fused: bool = False
    max_batch_size: Optional[int] = None
    tile_sizes: Optional[List[Tuple[int, int, int]]] = None

    def supports_precision(self, precision: str) -> bool:
        wanted = precision.lower()
        return any(wanted == p.lower() for p in self.precision_support)

    def supports_sm(self, sm_version: int) -> bool:
        return sm_version >= self.sm_version


# (name, backend, op, min sm, precisions, microscaling, fused, max batch, tiles)
_DEFAULT_TABLE = (
    ("cutlass_sm100_mxfp8_gemm", KernelBackend.CUTLASS, "gemm", 100, ["mxfp8", "e4m3", "e5m2"], True, True, None,
     [(256, 256, 128), (256, 192, 128), (128, 256, 128), (256, 128, 128), (128, 128, 128)]),
    ("cutlass_sm100_nvfp4_gemm", KernelBackend.CUTLASS, "gemm", 100, ["nvfp4", "mxfp4"], True, True, None,
     [(256, 128, 128), (128, 256, 128)]),
    ("cutlass_sm100_grouped_gemm_mxfp8", KernelBackend.CUTLASS, "grouped_gemm", 100, ["mxfp8"], True, True, 128,
     [(256, 256, 128), (128, 256, 128)]),
    ("cutlass_sm90_fp8_gemm", KernelBackend.CUTLASS, "gemm", 90, ["fp8", "e4m3", "e5m2"], False, True, None, None),
    ("te_mxfp8_linear", KernelBackend.TE, "linear", 90, ["mxfp8", "fp8", "fp16", "bf16"], True, True, None, None),
    ("te_attention", KernelBackend.TE, "attention", 80, ["fp16", "bf16", "fp8"], False, True, None, None),
    ("cublas_gemm", KernelBackend.CUBLAS, "gemm", 70, ["fp32", "fp16", "bf16"], False, False, None, None),
    ("cublas_grouped_gemm", KernelBackend.CUBLAS, "grouped_gemm", 70, ["fp32", "fp16", "bf16"], False, False, None, None),
    ("torch_linear", KernelBackend.TORCH, "linear", 0, ["fp32", "fp16", "bf16"], False, False, None, None),
    # the MX quantiser of this package (row-wise, column-wise, fused both-directions)
    ("sm100_mxfp8_quantize", KernelBackend.CUSTOM, "quantize", 100, ["mxfp8"], True, True, None, [(128, 128, 1)]),
)

# precisions tried, in order, when the wanted one has no kernel (registry.py:255-262 of the reference)
_WIDER = {
    "nvfp4": ["mxfp8", "fp8", "fp16", "bf16", "fp32"],
    "mxfp4": ["mxfp8", "fp8", "fp16", "bf16", "fp32"],
    "mxfp8": ["fp8", "fp16", "bf16", "fp32"],
    "fp8": ["fp16", "bf16", "fp32"],
    "fp16": ["bf16", "fp32"],
    "bf16": ["fp32"],
}


def _preference(spec: KernelSpec, prefer_fused: bool) -> int:
    """Blackwell first, then fused, then CUTLASS over TE, then microscaling (registry.py:209-221)."""
    score = 1000 if spec.sm_version >= 100 else 0
    if prefer_fused and spec.is_fused:
        score += 100
    score += {KernelBackend.CUTLASS: 50, KernelBackend.TE: 40}.get(spec.backend, 0)
    if spec.has_microscaling:
        score += 20
    return score


class KernelRegistry:
    def __init__(self) -> None:
        self.kernels: Dict[str, List[KernelSpec]] = {}
        for row in _DEFAULT_TABLE:
            self.register(KernelSpec(*row))

    def register(self, kernel: KernelSpec) -> None:
        self.kernels.setdefault(kernel.op_type, []).append(kernel)

    def find_kernel(self, op_type: str, precision: str, sm_version: int, prefer_fused: bool = True,
                    require_microscaling: bool = False) -> Optional[KernelSpec]:
        best, best_score = None, -1
        for spec in self.kernels.get(op_type, ()):
            if not (spec.supports_sm(sm_version) and spec.supports_precision(precision)):
                continue
            if require_microscaling and not spec.has_microscaling:
                continue
            score = _preference(spec, prefer_fused)
            if score > best_score:                    # first registered wins ties, as a stable sort would
                best, best_score = spec, score
        return best

    def find_fallback_chain(self, op_type: str, precision: str, sm_version: int) -> List[KernelSpec]:
        chain: List[KernelSpec] = []

        def push(spec: Optional[KernelSpec]) -> None:
            if spec is not None and spec not in chain:
                chain.append(spec)

        push(self.find_kernel(op_type, precision, sm_version))
        if precision in ("mxfp8", "nvfp4", "mxfp4"):
            push(self.find_kernel(op_type, "fp8", sm_version, require_microscaling=False))
        for wider in _WIDER.get(precision, ()):
            push(self.find_kernel(op_type, wider, sm_version))
        if op_type in ("gemm", "linear"):
            push(self.find_kernel("linear", "fp32", 0))
        return chain

    def get_kernel_info(self, kernel_name: str) -> Optional[KernelSpec]:
        for specs in self.kernels.values():
            for spec in specs:
                if spec.name == kernel_name:
                    return spec
        return None

    def list_kernels(self, op_type: Optional[str] = None) -> List[KernelSpec]:
        if op_type:
            return self.kernels.get(op_type, [])
        return [spec for specs in self.kernels.values() for spec in specs]

    def validate_for_hardware(self, sm_version: int) -> Dict[str, List[str]]:
        return {op: [s.name for s in specs if s.supports_sm(sm_version)] for op, specs in self.kernels.items()}


_global_registry = KernelRegistry()


def get_registry() -> KernelRegistry:
    return _global_registry


def register_kernel(kernel: KernelSpec) -> None:
    _global_registry.register(kernel)
