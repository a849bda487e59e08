"""Drop-in for the reference's extension module ``deepwell.cutlass_kernels``.

Same classes, method names and argument meaning as the pybind11 module defined in
csrc/python_bindings.cpp:258-319 of the reference (BlackwellGemmKernel,
BlackwellGroupedGemmKernel, MicroscaleManager, PrecisionType, profile_kernel), bound to
the sm_100a kernels of this package through the C ABI (include/dw_mxfp8.h).

Differences from the reference, all deliberate:
  * ``dtype="mxfp8"`` really quantises both operands to MXFP8 and runs the block-scaled
    tcgen05 GEMM (the reference runs a bf16 cuBLAS GEMM there, csrc/cutlass_kernels.cpp:173-204);
  * ``quantize_mxfp8`` returns ``torch.float8_e4m3fn`` codes and E8M0 ``uint8`` scales instead
    of truncated ``int8`` and ``float32`` (csrc/python_bindings.cpp:211-214);
  * ``b`` is honoured as a [K, N] tensor of any stride; the reference reads the storage of a
    transposed view as if it were contiguous (csrc/python_bindings.cpp:50-53, :100);
  * ``c`` takes part in ``alpha*A@B + beta*C`` as in the reference's Python module
    (src/deepwell/cutlass_kernels.py:28-32); the compiled reference ignores it;
  * no CPU path: CPU tensors raise, as the reference's TORCH_CHECKs do (:82-85).
"""
from __future__ import annotations

import enum
from typing import List, Optional, Sequence, Tuple

import torch

from . import _native as nv

# The reference's pure-Python stand-in sets this flag to True; a real extension has no such flag.
CUTLASS_PYTHON_FALLBACK = False

_DTYPE_STRINGS = ("fp32", "fp16", "bf16", "mxfp8", "nvfp4", "mxfp4")   # python_bindings.cpp:56-68
_TORCH_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


class PrecisionType(enum.IntEnum):
    """csrc/cutlass_kernels.h:28-40, exported at csrc/python_bindings.cpp:262-272."""
    FP32 = 0
    FP16 = 1
    BF16 = 2
    FP8_E4M3 = 3
    FP8_E5M2 = 4
    MXFP8 = 5
    NVFP4 = 6
    MXFP4 = 7
    INT8 = 8
    INT4 = 9


# Dense peaks used by get_expected_tflops (nominal B200 figures, TFLOP/s).
_NOMINAL_PEAK = {"fp32": 80.0, "fp16": 2250.0, "bf16": 2250.0, "mxfp8": 4500.0, "nvfp4": 9000.0, "mxfp4": 9000.0}


def _check_2d_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"Input {name} must be on CUDA")
    if t.dim() != 2:
        raise RuntimeError(f"Input {name} must be 2D")


def mxfp8_gemm_bf16(a: torch.Tensor, b_kn: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0,
                    beta: float = 0.0, bias: Optional[torch.Tensor] = None, scale_rule: int = nv.RULE_OCP_FLOOR,
                    plan: Optional[int] = None) -> torch.Tensor:
    """alpha * A[M,K] @ B[K,N] + beta * C (+ bias) with both operands quantised to MXFP8 along K.
    plan: the caller's own GEMM plan word (nv.plan_word); None = the process default."""
    a = a.to(torch.bfloat16)
    b_kn = b_kn.to(torch.bfloat16)
    a_codes, a_sf = nv.quantize(a, nv.DIR_ROW, scale_rule, nv.SF_TILED)
    if b_kn.stride(0) == 1 and b_kn.stride(1) == b_kn.shape[0]:
        # a transposed view of an [N, K] weight: its storage already is the K-major operand
        b_codes, b_sf = nv.quantize(b_kn.t(), nv.DIR_ROW, scale_rule, nv.SF_TILED)
    else:
        b_codes, b_sf = nv.quantize(b_kn.contiguous(), nv.DIR_COL_T, scale_rule, nv.SF_TILED)
    out = None
    if beta != 0.0:
        if c is None:
            raise RuntimeError("beta != 0 needs the C operand")
        out = c.to(torch.bfloat16).contiguous().clone()
    return nv.gemm(a_codes, a_sf, b_codes, b_sf, out=out, bias=bias, alpha=alpha, beta=beta, plan=plan)


_STACK_LIMIT = 20 << 20     # elements per expert weight above which the experts are quantised one launch each


def mxfp8_grouped_gemm_bf16(a_list: Sequence[torch.Tensor], b_list: Sequence[torch.Tensor], alpha: float = 1.0,
                            scale_rule: int = nv.RULE_OCP_FLOOR, weight_cache: Optional[dict] = None) -> List[torch.Tensor]:
    """[alpha * A_g[m_g,K] @ B_g[K,N] for g] in ONE GEMM launch when every group has the same K and N
    (the experts of an MoE layer): the activations are concatenated (each group padded with zero rows to a
    whole row tile) and quantised once, the weights are quantised into one stacked operand, and
    dw_mxfp8_gemm_grouped lets each row tile multiply its own group's weight.  Groups of different widths
    fall back to one launch per group.  Returns views into one output buffer.  `weight_cache` (a dict the caller
    keeps) lets repeated calls with unchanged weights reuse the stacked quantised operand: an entry is reused only
    when every weight is the same storage region (same storage object, offset, shape, strides, dtype, device) at the
    same version as when it was built.  The entry keeps the source tensors alive, so an address cannot be handed to
    a new tensor while the entry exists; weight lists rebuilt from temporaries on every call therefore never match
    a stale entry (they miss, and are quantised again)."""
    G = len(a_list)
    if G == 0:
        return []
    K, N = b_list[0].shape
    uniform = all(b.shape == (K, N) and a.dim() == 2 and a.shape[1] == K for a, b in zip(a_list, b_list))
    if not uniform or N % 128 or K % 32:
        return [mxfp8_gemm_bf16(a, b, None, alpha, 0.0, scale_rule=scale_rule) for a, b in zip(a_list, b_list)]
    dev = a_list[0].device
    sizes = [int(a.shape[0]) for a in a_list]
    rpt = 256 if sum(sizes) >= 512 * G else 128          # small groups: 128-row tiles waste less padding
    pieces, tile_group, offsets, row = [], [], [], 0
    for g, (a, m) in enumerate(zip(a_list, sizes)):
        padded = -(-m // rpt) * rpt
        offsets.append(row)
        pieces.append(a.to(torch.bfloat16))
        if padded != m:
            pieces.append(torch.zeros(padded - m, K, dtype=torch.bfloat16, device=dev))
        tile_group += [g] * (padded // rpt)
        row += padded
    if row == 0:
        return [torch.empty(0, N, dtype=torch.bfloat16, device=dev) for _ in a_list]
    a_codes, a_sf = nv.quantize(torch.cat(pieces, dim=0), nv.DIR_ROW, scale_rule, nv.SF_TILED)
    # weights: one stacked K-major operand [G * N, K] from one quantiser launch (N % 128 == 0, so every group owns
    # whole scale tiles and the stacked scale buffer is the concatenation of the groups' buffers)
    key = (G, K, N, scale_rule, str(dev)) + tuple(
        (b.untyped_storage().data_ptr(), b.storage_offset(), tuple(b.shape), tuple(b.stride()), b.dtype, b._version)
        for b in b_list)
    hit = False
    if weight_cache is not None and weight_cache.get("key") == key:
        held = weight_cache["sources"]
        # same storage OBJECTS as when the entry was built (they have been kept alive since, so equal addresses
        # cannot belong to recycled memory)
        hit = len(held) == G and all(h.untyped_storage()._cdata == b.untyped_storage()._cdata for h, b in zip(held, b_list))
    if hit:
        b_codes, b_sf = weight_cache["operand"]
    else:
        k_major = [b.stride(0) == 1 and b.stride(1) == K for b in b_list]     # transposed views of [N, K] weights
        if N * K > _STACK_LIMIT:
            # large experts: one quantiser launch per expert straight into its slice (stacking them first would
            # copy more bytes than the extra launches cost)
            b_codes = torch.empty(G * N, K, dtype=torch.uint8, device=dev)
            per_group = nv.scale_bytes(N, K, nv.SF_TILED)
            b_sf = torch.empty(G * per_group, dtype=torch.uint8, device=dev)
            for g, b in enumerate(b_list):
                bq = b.to(torch.bfloat16)
                nv.quantize_into(bq.t() if k_major[g] else bq.contiguous(), b_codes[g * N:(g + 1) * N],
                                 b_sf[g * per_group:(g + 1) * per_group], nv.DIR_ROW if k_major[g] else nv.DIR_COL_T,
                                 scale_rule, nv.SF_TILED)
        elif all(k_major):
            stacked = torch.cat([b.t() for b in b_list], dim=0).to(torch.bfloat16)
            b_codes, b_sf = nv.quantize(stacked, nv.DIR_ROW, scale_rule, nv.SF_TILED)
        else:
            stacked = torch.cat([b.to(torch.bfloat16) for b in b_list], dim=1)           # [K, G * N]
            b_codes, b_sf = nv.quantize(stacked, nv.DIR_COL_T, scale_rule, nv.SF_TILED)
        if weight_cache is not None:
            weight_cache["key"], weight_cache["operand"], weight_cache["sources"] = key, (b_codes, b_sf), list(b_list)
    groups = torch.tensor(tile_group, dtype=torch.int32).to(dev, non_blocking=True)
    d = nv.gemm_grouped(a_codes, a_sf, b_codes, b_sf, groups, G, rows_per_tile=rpt, alpha=alpha)
    return [d[o:o + m] for o, m in zip(offsets, sizes)]


class BlackwellGemmKernel:
    """csrc/python_bindings.cpp:35-113 (PyBlackwellGemmKernel)."""

    def __init__(self) -> None:
        nv.load()                      # fail now, loudly, if the native library is not built
        self.m = self.n = self.k = 0
        self.dtype = "bf16"
        self.use_microscaling = False
        self.block_size = 32
        self.tmem_residency = True
        self.cluster_shape: Optional[Tuple[int, int]] = None     # None: the kernel variant is chosen per problem
        self.plan = nv.plan_word(0)                               # this object's own launch choices (all automatic)
        self.initialized = False

    def initialize(self, m: int, n: int, k: int, dtype: str = "bf16", use_microscaling: bool = False,
                   block_size: int = 32) -> None:
        if dtype not in _DTYPE_STRINGS:
            dtype = "fp16"             # the reference's default for unknown strings (:56)
        if dtype in ("nvfp4", "mxfp4"):
            raise RuntimeError(f"dtype {dtype!r}: only the MXFP8 block-scaled kernel is built in this package")
        if dtype == "mxfp8" and block_size != 32:
            raise RuntimeError("MXFP8 uses 32-element scaling blocks")
        self.m, self.n, self.k = int(m), int(n), int(k)
        self.dtype, self.use_microscaling, self.block_size = dtype, bool(use_microscaling), int(block_size)
        self.initialized = True

    def gemm(self, a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0,
             beta: float = 0.0) -> torch.Tensor:
        _check_2d_cuda(a, "A")
        _check_2d_cuda(b, "B")
        if not self.initialized:
            raise RuntimeError("initialize() must be called before gemm()")
        if a.shape[0] != self.m or a.shape[1] != self.k or b.shape[0] != self.k or b.shape[1] != self.n:
            raise RuntimeError(f"operand shapes {tuple(a.shape)} x {tuple(b.shape)} do not match the initialised "
                               f"problem {self.m}x{self.n}x{self.k}")
        if self.dtype == "mxfp8":
            out = mxfp8_gemm_bf16(a, b, c, alpha, beta, plan=self.plan)
            return out if a.dtype == torch.bfloat16 else out.to(a.dtype)
        # plain library GEMM for the unquantised dtypes (the reference calls cuBLAS here, :143-172)
        td = _TORCH_DTYPES[self.dtype]
        d = torch.matmul(a.to(td), b.to(td))
        if alpha != 1.0:
            d = d * alpha
        if c is not None and beta != 0.0:
            d = d + beta * c.to(td)
        return d

    def enable_tmem_residency(self, enable: bool = True) -> None:
        # the accumulator always lives in TMEM in this kernel; the flag is kept for API parity
        self.tmem_residency = bool(enable)

    def set_cluster_shape(self, m: int, n: int) -> None:
        """(2, 1) pins THIS object's GEMMs to the CTA-pair kernel (cta_group::2, 256 x 256 tiles), (1, 1) to the
        single-CTA kernel (128 x 256 tiles).  The choice travels with every gemm() call of this object as its plan
        word; other kernel objects, DWLinear and other host threads are not affected.  Without a call the variant
        is chosen per problem."""
        if (m, n) not in ((1, 1), (2, 1)):
            raise RuntimeError("supported cluster shapes: (1, 1) and (2, 1)")
        self.cluster_shape = (int(m), int(n))
        self.plan = nv.plan_word(3 if m == 2 else 2)

    def get_expected_tflops(self) -> float:
        """Nominal dense peak of the selected precision (csrc/cutlass_kernels.cpp:233-263 kept hard-coded
        guesses; these are the published B200 dense figures) scaled by the same size heuristic."""
        peak = _NOMINAL_PEAK.get(self.dtype, 1000.0)
        eff = 0.8 if float(self.m) * self.n * self.k >= 1e9 else 0.5
        return peak * eff


class BlackwellGroupedGemmKernel:
    """csrc/python_bindings.cpp:116-194.  MXFP8 groups of equal K and N run as one grouped launch
    (mxfp8_grouped_gemm_bf16); the reference loops one cuBLAS call per group (csrc/cutlass_kernels.cpp:310-341)."""

    def __init__(self) -> None:
        nv.load()
        self.problem_sizes: List[Tuple[int, int, int]] = []
        self.dtype = "fp16"
        self.use_microscaling = False
        self.expert_parallel = True
        self._weight_cache: dict = {}

    def initialize(self, problem_sizes: Sequence[Tuple[int, int, int]], dtype: str = "fp16",
                   use_microscaling: bool = False) -> None:
        self.problem_sizes = [tuple(int(v) for v in p) for p in problem_sizes]
        self.dtype = dtype if dtype in _DTYPE_STRINGS else "fp16"
        self.use_microscaling = bool(use_microscaling)

    def grouped_gemm(self, a_list: Sequence[torch.Tensor], b_list: Sequence[torch.Tensor], alpha: float = 1.0,
                     beta: float = 0.0) -> List[torch.Tensor]:
        if len(a_list) != len(b_list):
            raise RuntimeError("a_list and b_list differ in length")
        for a, b in zip(a_list, b_list):
            if not a.is_cuda or not b.is_cuda:
                raise RuntimeError("All inputs must be on CUDA")
        if self.dtype == "mxfp8":
            outs = mxfp8_grouped_gemm_bf16(a_list, b_list, alpha, weight_cache=self._weight_cache)
            return [o if a.dtype == torch.bfloat16 else o.to(a.dtype) for o, a in zip(outs, a_list)]
        return [alpha * torch.matmul(a, b) for a, b in zip(a_list, b_list)]

    def set_expert_parallel_strategy(self, enable: bool) -> None:
        self.expert_parallel = bool(enable)


class MicroscaleManager:
    """csrc/python_bindings.cpp:197-241 (PyMicroscaleManager)."""

    def __init__(self) -> None:
        nv.load()

    def quantize_mxfp8(self, input: torch.Tensor, block_size: int = 32, direction: str = "row",
                       scale_layout: str = "flat", scale_rule: str = "ocp_floor"):
        """-> (codes float8_e4m3fn, scales uint8 E8M0).

        The two-argument call keeps the reference's meaning: blocks of 32 along the last
        dimension, codes shaped like the input, scales flat with one entry per block
        (csrc/python_bindings.cpp:206-214).  ``direction="col"`` scales along dim 0 and returns
        the payload transposed; ``scale_layout="tcgen05"`` returns the scales in the 512-byte
        tile layout the GEMM reads.
        """
        if not input.is_cuda:
            raise RuntimeError("Input must be on CUDA")
        if block_size != 32:
            raise RuntimeError("MXFP8 uses 32-element scaling blocks")
        x = input.to(torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x
        codes, scales = nv.quantize(x2, nv.DIRECTIONS[direction], nv.RULES[scale_rule], nv.LAYOUTS[scale_layout])
        if nv.DIRECTIONS[direction] == nv.DIR_ROW and input.dim() != 2:
            codes = codes.view(input.shape)
        if nv.LAYOUTS[scale_layout] == nv.SF_FLAT and direction == "row" and input.dim() != 2:
            scales = scales.reshape(-1)
        return codes, scales

    def dequantize_mxfp8(self, input: torch.Tensor, scales: torch.Tensor, block_size: int = 32,
                         scale_layout: str = "flat") -> torch.Tensor:
        """codes + scales -> bf16 (the kernel of the reference writes bf16 as well,
        csrc/mxfp8_quantization.cu:278, into a tensor its binding declared fp16, :230-232)."""
        if not input.is_cuda:
            raise RuntimeError("Input must be on CUDA")
        if not scales.is_cuda:
            raise RuntimeError("Scales must be on CUDA")
        if block_size != 32:
            raise RuntimeError("MXFP8 uses 32-element scaling blocks")
        codes2 = input.reshape(-1, input.shape[-1]) if input.dim() != 2 else input
        out = nv.dequantize(codes2.view(torch.uint8), scales.reshape(-1).view(torch.uint8), nv.LAYOUTS[scale_layout])
        return out.view(input.shape)


    def transpose_mxfp8(self, input: torch.Tensor, input_scales: torch.Tensor, block_size: int = 32,
                        scale_layout: str = "flat", scale_rule: str = "ocp_floor"):
        """Row-wise MX operand [rows, cols] -> the column-wise operand of the same values: payload transposed
        [cols, rows], scaling blocks along the former rows.  A transpose of MX data needs requantisation (the blocks
        change direction): dequantise, then quantise column-wise.  MicroscaleManager::transpose_mxfp8 of the reference
        (csrc/cutlass_kernels.cpp:412-424) is an empty body.  When the bf16 source is at hand, quantize_both gives
        both forms from one read and without the intermediate rounding."""
        if block_size != 32:
            raise RuntimeError("MXFP8 uses 32-element scaling blocks")
        x = self.dequantize_mxfp8(input, input_scales, block_size, scale_layout)
        x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x
        return nv.quantize(x2, nv.DIR_COL_T, nv.RULES[scale_rule], nv.LAYOUTS[scale_layout])

    def update_amax_history(self, tensor: torch.Tensor, amax_history: torch.Tensor) -> torch.Tensor:
        """Shifts ``amax_history`` (float32 [history_len], on the tensor's device) by one and stores max |tensor| at [0]
        (MicroscaleManager::update_amax_history, csrc/cutlass_kernels.cpp:426-434, empty in the reference)."""
        if not tensor.is_cuda:
            raise RuntimeError("Input must be on CUDA")
        nv.update_amax_history(tensor.to(torch.bfloat16).contiguous(), amax_history)
        return amax_history


def profile_kernel(kernel: BlackwellGemmKernel, warmup_iterations: int = 10, profile_iterations: int = 100) -> dict:
    """Times kernel.gemm on random operands with CUDA events (the reference returns constants,
    csrc/python_bindings.cpp:244-255)."""
    if not kernel.initialized:
        raise RuntimeError("initialize() must be called before profile_kernel()")
    dev = torch.device("cuda", torch.cuda.current_device())
    td = torch.bfloat16 if kernel.dtype == "mxfp8" else _TORCH_DTYPES[kernel.dtype]
    a = torch.randn(kernel.m, kernel.k, device=dev, dtype=td)
    b = torch.randn(kernel.k, kernel.n, device=dev, dtype=td)
    for _ in range(max(1, warmup_iterations)):
        kernel.gemm(a, b)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(max(1, profile_iterations)):
        kernel.gemm(a, b)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / max(1, profile_iterations)
    flops = 2.0 * kernel.m * kernel.n * kernel.k
    bytes_moved = (kernel.m * kernel.k + kernel.k * kernel.n + kernel.m * kernel.n) * a.element_size()
    return {"runtime_ms": ms, "tflops": flops / ms / 1e9, "memory_bandwidth_gb_s": bytes_moved / ms / 1e6,
            "expected_tflops": kernel.get_expected_tflops()}
