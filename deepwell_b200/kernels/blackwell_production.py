"""The linear-path classes of the reference's ``deepwell.kernels.blackwell_production`` over the MXFP8 kernels.

Kept: BlackwellConfig (src/deepwell/kernels/blackwell_production.py:50-77, the fields this path reads),
BlackwellGEMM.gemm with optional bias and activation fused into the GEMM epilogue (:189-229),
BlackwellGroupedGEMM (:232-276), FusedLinearGELU (:487-527), FusedLayerNormLinear (:530-575) and
optimize_model_for_blackwell (:578-624).  The attention classes of that module (BlackwellFlashAttention,
DWSelfAttention) belong to a different path and are not part of this package.

In the reference the fusion flags select arguments of a CUTLASS plan that is never built on a machine without the
CUTLASS Python package; here ``activation`` reaches dw_mxfp8_gemm_fused, which applies bias and ReLU / exact GELU / SiLU
to the fp32 accumulator before the bf16 rounding.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native as nv
from ..cutlass_kernels import mxfp8_gemm_bf16, mxfp8_grouped_gemm_bf16
from ..linear import DWLinear

_ACTIVATIONS = {None: "none", "none": "none", "relu": "relu", "gelu": "gelu", "silu": "silu", "swish": "silu"}


@dataclasses.dataclass
class BlackwellConfig:
    sm_version: int = 100
    use_mxfp8: bool = True
    use_fp4: bool = False
    use_tcgen05: bool = True
    preferred_cluster_size: int = 2
    fuse_gelu: bool = True
    fuse_layernorm: bool = True
    fuse_bias: bool = True
    persistent_kernel: bool = True


class BlackwellGEMM:
    """gemm(a [M,K], b [K,N], bias, activation) -> bf16 [M,N]; operands are quantised to MXFP8 along K."""

    def __init__(self, config: Optional[BlackwellConfig] = None):
        nv.ext()
        self.config = config or BlackwellConfig()
        if self.config.use_fp4:
            raise RuntimeError("only the MXFP8 block-scaled kernel is built in this package")

    def gemm(self, a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
             activation: Optional[str] = None) -> torch.Tensor:
        if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
            raise RuntimeError(f"Dimension mismatch: {tuple(a.shape)} x {tuple(b.shape)}")
        if not a.is_cuda or not b.is_cuda:
            raise RuntimeError("inputs must be on CUDA")
        act = _ACTIVATIONS.get(activation)
        if act is None:
            raise RuntimeError(f"unknown activation {activation!r}")
        bias_b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        fuse_act = act != "none" and (act != "gelu" or self.config.fuse_gelu)
        if not fuse_act and (bias_b is None or self.config.fuse_bias):
            out = mxfp8_gemm_bf16(a, b, None, 1.0, 0.0, bias=bias_b)
        else:
            a_codes, a_sf = nv.quantize(a.to(torch.bfloat16), nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
            bb = b.to(torch.bfloat16)
            if bb.stride(0) == 1 and bb.stride(1) == bb.shape[0]:
                b_codes, b_sf = nv.quantize(bb.t(), nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
            else:
                b_codes, b_sf = nv.quantize(bb.contiguous(), nv.DIR_COL_T, nv.RULE_OCP_FLOOR, nv.SF_TILED)
            fused_bias = bias_b if self.config.fuse_bias else None
            out, _, _ = nv.gemm_fused(a_codes, a_sf, b_codes, b_sf, bias=fused_bias,
                                      activation=act if fuse_act and fused_bias is bias_b else "none", quantize_out=False)
            if fused_bias is None and bias_b is not None:      # bias outside the kernel: the activation follows it
                out = out + bias_b
                if fuse_act:
                    out = getattr(F, act)(out)
        if act != "none" and not fuse_act:
            out = getattr(F, act)(out)
        return out


class BlackwellGroupedGEMM:
    """grouped_gemm(inputs, weights): one launch for groups of equal K and N (the experts of an MoE layer)."""

    def __init__(self, config: Optional[BlackwellConfig] = None):
        nv.ext()
        self.config = config or BlackwellConfig()
        self._weight_cache: dict = {}

    def grouped_gemm(self, inputs: Sequence[torch.Tensor], weights: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        if len(inputs) != len(weights):
            raise RuntimeError("inputs and weights differ in length")
        return mxfp8_grouped_gemm_bf16(inputs, weights, 1.0, weight_cache=self._weight_cache)


class FusedLinearGELU(nn.Module):
    """Linear + exact GELU.  Without autograd the bias and the GELU run in the GEMM epilogue on the fp32 accumulator
    (one kernel after the quantiser); with autograd the layer is DWLinear followed by F.gelu, whose backward needs the
    pre-activation the fused kernel does not keep."""

    def __init__(self, in_features: int, out_features: int, config: Optional[BlackwellConfig] = None):
        super().__init__()
        self.config = config or BlackwellConfig()
        self.linear = DWLinear(in_features, out_features, bias=True, dtype=torch.bfloat16)
        nn.init.xavier_uniform_(self.linear.weight)
        nn.init.zeros_(self.linear.bias)
        self.in_features, self.out_features = in_features, out_features

    @property
    def weight(self) -> nn.Parameter:
        return self.linear.weight

    @property
    def bias(self) -> nn.Parameter:
        return self.linear.bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("FusedLinearGELU runs on CUDA (sm_100a) only; there is no CPU path")
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad or self.bias.requires_grad)
        if needs_grad or not self.config.fuse_gelu:
            return F.gelu(self.linear(x))
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features).to(torch.bfloat16)
        (w_codes, w_sf), _ = self.linear._quantized_weight(need_col=False)
        x_codes, x_sf = nv.quantize(x2d, nv.DIR_ROW, self.linear.scale_rule, nv.SF_TILED)
        y, _, _ = nv.gemm_fused(x_codes, x_sf, w_codes, w_sf, bias=self.bias.detach().to(torch.bfloat16).contiguous(),
                                activation="gelu", quantize_out=False)
        return y.reshape(*lead, self.out_features).to(x.dtype)


class FusedMLP(nn.Module):
    """up-projection -> activation -> down-projection.  Without autograd the hidden activation never exists in bf16:
    the first GEMM's epilogue applies bias and activation to the fp32 accumulator and writes the result already
    quantised (E4M3 codes + tiled E8M0 scales, bit-identical to quantising the bf16 result), and the second GEMM
    consumes it as its A operand.  With autograd the three steps run separately (DWLinear, torch activation, DWLinear).
    The reference runs its MLP as two GEMM calls with torch's GELU in between (src/deepwell/engine.py:132-209)."""

    def __init__(self, in_features: int, hidden_features: int, out_features: Optional[int] = None,
                 activation: str = "gelu", bias: bool = True, config: Optional[BlackwellConfig] = None):
        super().__init__()
        if _ACTIVATIONS.get(activation) in (None, "none"):
            raise ValueError(f"activation must be one of relu, gelu, silu; got {activation!r}")
        self.config = config or BlackwellConfig()
        self.activation = _ACTIVATIONS[activation]
        self.up = DWLinear(in_features, hidden_features, bias=bias, dtype=torch.bfloat16)
        self.down = DWLinear(hidden_features, out_features or in_features, bias=bias, dtype=torch.bfloat16)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("FusedMLP runs on CUDA (sm_100a) only; there is no CPU path")
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            return self.down(getattr(F, self.activation)(self.up(x)))
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.up.in_features).to(torch.bfloat16)
        (uw, us), _ = self.up._quantized_weight(need_col=False)
        (dw_, ds), _ = self.down._quantized_weight(need_col=False)
        bf16 = lambda p: None if p is None else p.detach().to(torch.bfloat16).contiguous()
        xc, xs = nv.quantize(x2d, nv.DIR_ROW, self.up.scale_rule, nv.SF_TILED)
        _, hc, hs = nv.gemm_fused(xc, xs, uw, us, bias=bf16(self.up.bias), activation=self.activation, quantize_out=True,
                                  write_d=False, rule=self.up.scale_rule)
        y = nv.gemm(hc, hs, dw_, ds, bias=bf16(self.down.bias))
        return y.reshape(*lead, self.down.out_features).to(x.dtype)


class FusedSwiGLUMLP(nn.Module):
    """The gated MLP of Llama-style models: down(silu(gate(x)) * up(x)), parameters named as in those models
    (gate_proj, up_proj, down_proj; no biases).

    Without autograd the whole block is one quantiser launch and two GEMMs.  gate and up are one GEMM against their
    weights interleaved in groups of 32 rows, whose epilogue (DW_ACT_SWIGLU) forms silu(gate) * up from the fp32
    accumulators, rounds to bf16 once and writes the result already quantised as the down projection's A operand:
    neither the [tokens, 2 F] gate/up activations nor the [tokens, F] product ever exist in bf16 in memory, and the
    quantiser pass over the largest activation of the block is gone.  With autograd the three DWLinear layers run
    separately (the backward of the gated unit needs gate and up).  ``fuse=False`` forces that path for comparison.
    Gives EpilogueConfig::Op::BiasSwish (csrc/cutlass_kernels.h:65-77 of the reference, declared and never applied) the
    gated form this model family needs."""

    def __init__(self, hidden_size: int, intermediate_size: int, config: Optional[BlackwellConfig] = None, fuse: bool = True):
        super().__init__()
        if hidden_size % 32 or intermediate_size % 32:
            raise ValueError("hidden_size and intermediate_size must be multiples of 32 (the MX block size)")
        self.config = config or BlackwellConfig()
        self.fuse = fuse
        self.gate_proj = DWLinear(hidden_size, intermediate_size, bias=False, dtype=torch.bfloat16)
        self.up_proj = DWLinear(hidden_size, intermediate_size, bias=False, dtype=torch.bfloat16)
        self.down_proj = DWLinear(intermediate_size, hidden_size, bias=False, dtype=torch.bfloat16)
        self._gu_key = None
        self._gu_operand = None            # interleaved gate+up weight, quantised (persistent buffers)

    def _gate_up_operand(self):
        g, u = self.gate_proj.weight, self.up_proj.weight
        key = (g.data_ptr(), g._version, u.data_ptr(), u._version, g.device)
        if key != self._gu_key or self._gu_operand is None:
            fused = nv.interleave_gate_up(g.detach().to(torch.bfloat16), u.detach().to(torch.bfloat16)).contiguous()
            if self._gu_operand is None or self._gu_operand[0].device != fused.device:
                n, k = fused.shape
                self._gu_operand = (torch.empty(n, k, dtype=torch.uint8, device=fused.device),
                                    torch.empty(nv.scale_bytes(n, k, nv.SF_TILED), dtype=torch.uint8, device=fused.device))
            nv.quantize_into(fused, self._gu_operand[0], self._gu_operand[1], nv.DIR_ROW, self.gate_proj.scale_rule, nv.SF_TILED)
            self._gu_key = key
        return self._gu_operand

    def invalidate_weight_cache(self) -> None:
        """After a write through ``weight.data`` (see DWLinear.invalidate_weight_cache)."""
        self._gu_key = None
        for m in (self.gate_proj, self.up_proj, self.down_proj):
            m.invalidate_weight_cache()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("FusedSwiGLUMLP runs on CUDA (sm_100a) only; there is no CPU path")
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters()))
        if needs_grad or not self.fuse:
            return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.gate_proj.in_features).to(torch.bfloat16)
        gu_codes, gu_sf = self._gate_up_operand()
        (dw_, ds), _ = self.down_proj._quantized_weight(need_col=False)
        xc, xs = nv.quantize(x2d, nv.DIR_ROW, self.gate_proj.scale_rule, nv.SF_TILED)
        _, hc, hs = nv.gemm_fused(xc, xs, gu_codes, gu_sf, activation="swiglu", quantize_out=True, write_d=False,
                                  rule=self.gate_proj.scale_rule)
        y = nv.gemm(hc, hs, dw_, ds)
        return y.reshape(*lead, self.down_proj.out_features).to(x.dtype)


class FusedLayerNormLinear(nn.Module):
    """LayerNorm followed by an MXFP8 linear layer.  The normalisation is torch's; the linear layer is DWLinear (the
    reference's class of this name computes both with torch, src/deepwell/kernels/blackwell_production.py:554-575)."""

    def __init__(self, normalized_shape: int, out_features: int, config: Optional[BlackwellConfig] = None):
        super().__init__()
        self.config = config or BlackwellConfig()
        self.norm = nn.LayerNorm(normalized_shape, dtype=torch.bfloat16)
        self.linear = DWLinear(normalized_shape, out_features, bias=True, dtype=torch.bfloat16)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear(self.norm(x))


def optimize_model_for_blackwell(model: nn.Module, config: Optional[BlackwellConfig] = None) -> nn.Module:
    """Every eligible nn.Linear of ``model`` becomes a DWLinear, in place (the reference's function of this name also
    swaps attention modules, which are outside this package)."""
    from ..optimizer import optimize
    config = config or BlackwellConfig()
    return optimize(model, precision="mxfp8" if config.use_mxfp8 else "bf16", verbose=False, inplace=True)
