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
        """One call into deepwell_b200._C: the autograd node (MXFP8LinearFunction of csrc/python_bindings.cpp) quantises
        x, runs the GEMM and, in backward, quantises dY and runs the two gradient GEMMs, all without re-entering
        Python.  The node keeps references to this module's weight operand buffers, not copies: a backward sees the
        weight as it was last quantised, which is the forward's weight in any loop that does not update the weight
        between a forward and its backward."""
        if not x.is_cuda:
            raise RuntimeError("DWLinear runs on CUDA (sm_100a) only; there is no CPU path")
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features)
        grad = torch.is_grad_enabled()
        (w_codes, w_sf), w_col = self._quantized_weight(need_col=grad and x2d.requires_grad)
        y = nv.ext().linear(x2d, self.weight, self.bias, w_codes, w_sf, None if w_col is None else w_col[0],
                            None if w_col is None else w_col[1], self.scale_rule, nv.status_word(x.device), _CHECK_STATUS)
        if _CHECK_STATUS and not y.requires_grad:
            nv.check_status(x.device)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, mxfp8"
