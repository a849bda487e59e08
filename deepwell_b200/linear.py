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
import torch.nn.functional as F

from . import _native as nv


def _pad_rows_to_32(t: torch.Tensor) -> torch.Tensor:
    m = t.shape[0]
    pad = (-m) % 32
    return t if pad == 0 else F.pad(t, (0, 0, 0, pad))


class _MXFP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], module: "DWLinear"):
        need_x_grad, need_w_grad = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        w_row, w_col = module._quantized_weight(need_col=need_x_grad)
        xb = x2d.to(torch.bfloat16)
        m = xb.shape[0]
        if need_w_grad:
            xp = _pad_rows_to_32(xb)
            xr_c, xr_s, xc_c, xc_s = nv.quantize_both(xp, module.scale_rule, nv.SF_TILED)
            x_col = (xc_c, xc_s)
        else:
            xp = xb
            xr_c, xr_s = nv.quantize(xb, nv.DIR_ROW, module.scale_rule, nv.SF_TILED)
            x_col = None
        bias_b = None if bias is None else bias.to(torch.bfloat16)
        y = nv.gemm(xr_c, xr_s, w_row[0], w_row[1], bias=bias_b)
        if y.shape[0] != m:
            y = y[:m]
        ctx.module = module
        ctx.m = m
        ctx.x_dtype, ctx.w_dtype = x2d.dtype, weight.dtype
        ctx.has_bias = bias is not None
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.x_col = x_col
        ctx.w_col = w_col
        return y if x2d.dtype == torch.bfloat16 else y.to(x2d.dtype)

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        module = ctx.module
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dyb = _pad_rows_to_32(dy.to(torch.bfloat16).contiguous())
        dx = dw = db = None
        if need_dw:
            dr_c, dr_s, dc_c, dc_s = nv.quantize_both(dyb, module.scale_rule, nv.SF_TILED)
        else:
            dr_c, dr_s = nv.quantize(dyb, nv.DIR_ROW, module.scale_rule, nv.SF_TILED)
        if need_dx:
            w_col = ctx.w_col if ctx.w_col is not None else module._quantized_weight(need_col=True)[1]
            dx = nv.gemm(dr_c, dr_s, w_col[0], w_col[1])[: ctx.m]
            if ctx.x_dtype != torch.bfloat16:
                dx = dx.to(ctx.x_dtype)
        if need_dw:
            xc_c, xc_s = ctx.x_col
            dw = nv.gemm(dc_c, dc_s, xc_c, xc_s)
            if ctx.w_dtype != torch.bfloat16:
                dw = dw.to(ctx.w_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(dim=0).to(ctx.bias_dtype)
        return dx, dw, db, None


class DWLinear(nn.Module):
    """Drop-in for nn.Linear (same parameter names, so state_dicts interchange)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 scale_rule: str = "ocp_floor"):
        super().__init__()
        if in_features % 32 or out_features % 32:
            raise ValueError("DWLinear needs in_features and out_features to be multiples of 32 (the MX block size)")
        nv.load()
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
        nv.load()
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
