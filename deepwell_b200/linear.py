"""DWLinear — nn.Linear whose three GEMMs (forward, dgrad, wgrad) run in MXFP8 on sm_100a.

The reference reserves the place for this module (src/deepwell/optimizer.py:206-212 prints
"Linear (MXFP8 coming soon)") and has one linear replacement, OptimizedLinear
(src/deepwell/kernels/production_kernels.py:145-194), whose conventions are kept: inputs of
any rank are flattened to [tokens, in_features], bias is added after the GEMM, weight is
[out_features, in_features].  OptimizedLinear has no autograd function; this one does.

Scaling blocks always run along the contraction dimension of the GEMM that consumes the
operand, so every tensor is needed in two quantised forms:

    forward  Y[M,N]  = X[M,K]  . W[N,K]^T    X row-wise,  W row-wise          (contract K)
    dgrad    dX[M,K] = dY[M,N] . W[N,K]      dY row-wise, W column-wise^T     (contract N)
    wgrad    dW[N,K] = dY^T    . X           dY column-wise^T, X column-wise^T (contract M)

X, dY and W are each read once by the fused both-directions quantiser.  The quantised forms
of W are cached until the parameter changes.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _native as nv


class _MXFP8LinearFn(torch.autograd.Function):
    """One call into deepwell_b200._C per direction (linear_forward / linear_backward of
    csrc/python_bindings.cpp): the quantiser and GEMM launches and their output allocations happen
    there, so the host cost per layer is one Python->C++ transition each way."""

    @staticmethod
    def forward(ctx, x2d: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], module: "DWLinear"):
        need_x_grad, need_w_grad = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        w_row, w_col = module._quantized_weight(need_col=need_x_grad)
        bf16 = torch.bfloat16
        xb = x2d if x2d.dtype is bf16 else x2d.to(bf16)
        bias_b = bias if bias is None or bias.dtype is bf16 else bias.to(bf16)
        y, xc_c, xc_s = nv.ext().linear_forward(xb, w_row[0], w_row[1], bias_b, need_w_grad, module.scale_rule,
                                                nv.status_word(xb.device))
        ctx.module = module
        ctx.m = xb.shape[0]
        ctx.x_dtype, ctx.w_dtype = x2d.dtype, weight.dtype
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.x_col = (xc_c, xc_s) if need_w_grad else None
        ctx.w_col = w_col
        return y if x2d.dtype is bf16 else y.to(x2d.dtype)

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        module = ctx.module
        need_dx, need_dw, need_db = ctx.needs_input_grad[:3]
        bf16 = torch.bfloat16
        dyb = dy if dy.dtype is bf16 else dy.to(bf16)
        w_cc = w_cs = x_cc = x_cs = None
        if need_dx:
            w_cc, w_cs = ctx.w_col if ctx.w_col is not None else module._quantized_weight(need_col=True)[1]
        if need_dw:
            x_cc, x_cs = ctx.x_col
        need_db = need_db and ctx.bias_dtype is not None
        db_mode = 0 if not need_db else (1 if ctx.bias_dtype is bf16 else 2)       # bf16 sums only for a bf16 bias
        dx, dw, db = nv.ext().linear_backward(dyb, w_cc, w_cs, x_cc, x_cs, ctx.m, module.scale_rule, db_mode,
                                              nv.status_word(dyb.device))
        if need_dx and ctx.x_dtype is not bf16:
            dx = dx.to(ctx.x_dtype)
        if need_dw and ctx.w_dtype is not bf16:
            dw = dw.to(ctx.w_dtype)
        if need_db and db.dtype is not ctx.bias_dtype:
            db = db.to(ctx.bias_dtype)
        return dx, dw, db, None


class DWLinear(nn.Module):
    """Drop-in for nn.Linear (same parameter names, so state_dicts interchange)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 scale_rule: str = "ocp_floor"):
        super().__init__()
        if in_features % 32 or out_features % 32:
            raise ValueError("DWLinear needs in_features and out_features to be multiples of 32 (the MX block size)")
        nv.ext()
        self.in_features, self.out_features = in_features, out_features
        kw = {"device": device, "dtype": dtype}
        self.weight = nn.Parameter(torch.empty(out_features, in_features, **kw))
        self.bias = nn.Parameter(torch.empty(out_features, **kw)) if bias else None
        self.scale_rule = nv.RULES[scale_rule]
        self._wq_key: Optional[Tuple] = None
        self._wq_row = None
        self._wq_col = None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        if self.bias is not None:
            bound = 1.0 / self.in_features ** 0.5
            nn.init.uniform_(self.bias, -bound, bound)

    @classmethod
    def from_linear(cls, linear: nn.Linear, scale_rule: str = "ocp_floor") -> "DWLinear":
        """Shares the nn.Linear's parameters (no copy), as optimize_model_inplace does
        (src/deepwell/kernels/production_kernels.py:382-384)."""
        mod = cls.__new__(cls)
        nn.Module.__init__(mod)
        if linear.in_features % 32 or linear.out_features % 32:
            raise ValueError("DWLinear needs in_features and out_features to be multiples of 32")
        nv.ext()
        mod.in_features, mod.out_features = linear.in_features, linear.out_features
        mod.weight = linear.weight
        mod.bias = linear.bias
        mod.scale_rule = nv.RULES[scale_rule]
        mod._wq_key, mod._wq_row, mod._wq_col = None, None, None
        return mod

    def _quantized_weight(self, need_col: bool):
        """(row-wise operand, column-wise transposed operand) of the weight; cached per version."""
        w = self.weight
        key = (w.data_ptr(), w._version, w.device, w.dtype)
        if key != self._wq_key or (need_col and self._wq_col is None):
            wb = w.detach().to(torch.bfloat16).contiguous()
            if need_col:
                rc, rs, cc, cs = nv.quantize_both(wb, self.scale_rule, nv.SF_TILED)
                self._wq_row, self._wq_col = (rc, rs), (cc, cs)
            else:
                self._wq_row, self._wq_col = nv.quantize(wb, nv.DIR_ROW, self.scale_rule, nv.SF_TILED), None
            self._wq_key = key
        return self._wq_row, self._wq_col

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("DWLinear runs on CUDA (sm_100a) only; there is no CPU path")
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features)
        y = _MXFP8LinearFn.apply(x2d, self.weight, self.bias, self)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, mxfp8"
