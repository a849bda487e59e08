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

X, dY and W are each read once by the fused both-directions quantiser.

The quantised forms of W live in buffers the module keeps for its whole life and are refreshed
when the parameter's version counter moves (every in-place update an optimizer makes moves it).
Two cases need more than that, and get it:
  * while a CUDA graph is being captured the weight is ALWAYS re-quantised, into those same
    buffers, so the launch is part of the graph: a replay after an optimizer step sees the new
    weight, and the addresses the graph recorded stay valid;
  * a write through ``weight.data`` (master-weight optimizers, EMA swaps, ``p.data.clamp_()``)
    does not move the version counter.  Call ``invalidate_weight_cache()`` after such a write, or
    construct / set the module with ``weight_cache="off"`` to quantise on every forward.
"""
from __future__ import annotations

from typing import Optional, Tuple

import os

import torch
import torch.nn as nn

from . import _native as nv

# DW_CHECK_STATUS=1: every DWLinear forward (outside autograd) and backward ends by synchronising and reading the
# status word the kernels set when a bounded wait expires (nv.check_status raises).  Off by default because of the
# synchronisation; without it, poll nv.check_status() yourself where the training loop synchronises anyway.
_CHECK_STATUS = os.environ.get("DW_CHECK_STATUS", "0") not in ("", "0")


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
        if _CHECK_STATUS and not (need_x_grad or need_w_grad):
            nv.check_status(xb.device)
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
        if _CHECK_STATUS:
            nv.check_status(dyb.device)
        return dx, dw, db, None


class DWLinear(nn.Module):
    """Drop-in for nn.Linear (same parameter names, so state_dicts interchange)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 scale_rule: str = "ocp_floor", weight_cache: str = "version"):
        super().__init__()
        if in_features % 32 or out_features % 32:
            raise ValueError("DWLinear needs in_features and out_features to be multiples of 32 (the MX block size)")
        nv.ext()
        self.in_features, self.out_features = in_features, out_features
        kw = {"device": device, "dtype": dtype}
        self.weight = nn.Parameter(torch.empty(out_features, in_features, **kw))
        self.bias = nn.Parameter(torch.empty(out_features, **kw)) if bias else None
        self.scale_rule = nv.RULES[scale_rule]
        self._init_weight_cache(weight_cache)
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
        mod._init_weight_cache("version")
        return mod

    def _init_weight_cache(self, mode: str) -> None:
        if mode not in ("version", "off"):
            raise ValueError("weight_cache must be 'version' or 'off'")
        self.weight_cache = mode
        self._wq_key: Optional[Tuple] = None      # what the buffers were last filled from
        self._wq_has_col = False                  # whether that fill included the column-wise form
        self._wq_row = None                       # (codes [N, K], tiled scales): persistent buffers
        self._wq_col = None                       # (codes [K, N], tiled scales): persistent buffers

    def invalidate_weight_cache(self) -> None:
        """Forces the next forward to quantise the weight again.  Needed after a write that does not move
        ``weight._version``, i.e. any write through ``weight.data``."""
        self._wq_key = None

    def _weight_buffers(self, need_col: bool):
        """The module's own operand buffers; allocated once per (device, shape) and never replaced, so pointers a
        captured graph recorded stay valid and stay the module's."""
        w = self.weight
        n, k = w.shape
        if self._wq_row is None or self._wq_row[0].device != w.device or tuple(self._wq_row[0].shape) != (n, k):
            u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=w.device)
            self._wq_row = (u8(n, k), u8(nv.scale_bytes(n, k, nv.SF_TILED)))
            self._wq_col, self._wq_key = None, None
        if need_col and self._wq_col is None:
            u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=w.device)
            self._wq_col = (u8(k, n), u8(nv.scale_bytes(k, n, nv.SF_TILED)))
            self._wq_key = None
        return self._wq_row, (self._wq_col if need_col else None)

    def _quantized_weight(self, need_col: bool):
        """(row-wise operand, column-wise transposed operand or None) of the weight, in the module's persistent
        buffers.  Refilled when the parameter's (storage, version) changed, always while a CUDA graph is being
        captured, and always with ``weight_cache="off"``."""
        w = self.weight
        row, col = self._weight_buffers(need_col)
        key = (w.data_ptr(), w._version, w.device, w.dtype)
        capturing = w.is_cuda and torch.cuda.is_current_stream_capturing()
        if capturing or self.weight_cache == "off" or key != self._wq_key or (need_col and not self._wq_has_col):
            wb = w.detach()
            if wb.dtype is not torch.bfloat16:
                wb = wb.to(torch.bfloat16)
            wb = wb.contiguous()
            nv.ext().quantize_both_into(wb, row[0], row[1], None if col is None else col[0], None if col is None else col[1],
                                        self.scale_rule)
            self._wq_key, self._wq_has_col = key, col is not None
        return row, col

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("DWLinear runs on CUDA (sm_100a) only; there is no CPU path")
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features)
        y = _MXFP8LinearFn.apply(x2d, self.weight, self.bias, self)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, mxfp8"
