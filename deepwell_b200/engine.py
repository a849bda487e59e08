"""The MLP executor of the reference's ``deepwell.engine`` over the MXFP8 kernels.

The reference's ExecutableModel (src/deepwell/engine.py:17-315) is an execution engine around a compiled IR; of it
only ``_mlp_with_cutlass`` (:132-209) is a caller of the linear hot path, and it is the one method kept here, with its
signature: ``_mlp_with_cutlass(x, mlp, layer_idx)`` walks the layers of an MLP (``nn.Linear``, activation modules, anything
else) over a [batch, seq, hidden] activation.  In the reference every Linear becomes one ``CutlassKernel.gemm`` on a
``weight.t().contiguous()`` copy made on every call, with the comment "skip quantization and use BF16 directly"
(:163-165), a separate bias add and torch's GELU in between.  Here

  * a ``Linear -> ReLU/GELU/SiLU -> Linear`` run is two GEMMs: bias, activation and the quantisation of the hidden
    activation happen in the first GEMM's epilogue (dw_mxfp8_gemm_fused), the second GEMM consumes the codes;
  * any other Linear is quantise + block-scaled GEMM with the bias in the epilogue;
  * quantised weights are kept per layer until the parameter changes (no per-call transpose or copy).

``forward`` of ExecutableModel runs the original model: the IR-driven engine around it is outside this package.
No autograd (the reference's method has none either: its extension returns tensors without grad_fn).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import _native as nv

_ACT_MODULES = {nn.ReLU: "relu", nn.GELU: "gelu", nn.SiLU: "silu"}


class ExecutableModel(nn.Module):
    def __init__(self, engine=None, original_model: Optional[nn.Module] = None):
        super().__init__()
        nv.ext()
        self.engine = engine
        self.original_model = original_model
        self.use_cutlass = True
        self.kernel_cache: Dict[str, Tuple] = {}       # "mlp_linear_{layer_idx}_{i}" -> (key, (codes, tiled scales))

    def forward(self, *inputs):
        if self.original_model is None:
            raise RuntimeError("no model to run")
        return self.original_model(*inputs)

    def _weight_operand(self, name: str, layer: nn.Linear):
        w = layer.weight
        key = (w.data_ptr(), w._version, w.device, w.dtype, tuple(w.shape))
        hit = self.kernel_cache.get(name)
        if hit is None or hit[0] != key:
            hit = (key, nv.quantize(w.detach().to(torch.bfloat16).contiguous(), nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED), w)
            self.kernel_cache[name] = hit               # the entry keeps `w` alive, so its address cannot be reused
        return hit[1]

    @torch.no_grad()
    def _mlp_with_cutlass(self, x: torch.Tensor, mlp, layer_idx: int) -> torch.Tensor:
        """x [batch, seq, hidden] (or any [..., hidden]) through the layers of `mlp`, MXFP8 for every nn.Linear whose
        feature counts are multiples of 32; other layers run as they are."""
        if not x.is_cuda:
            raise RuntimeError("_mlp_with_cutlass runs on CUDA (sm_100a) only; there is no CPU path")
        lead, out_dtype = x.shape[:-1], x.dtype
        layers = list(mlp)
        h = x.reshape(-1, x.shape[-1])
        codes = sf = None                                # h already quantised by the previous GEMM's epilogue
        i = 0
        bf16 = lambda t: None if t is None else t.detach().to(torch.bfloat16).contiguous()
        while i < len(layers):
            layer = layers[i]
            eligible = isinstance(layer, nn.Linear) and layer.in_features % 32 == 0 and layer.out_features % 32 == 0
            if not eligible:
                h = layer(h)
                i += 1
                continue
            if codes is None:
                codes, sf = nv.quantize(h.to(torch.bfloat16).contiguous(), nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
            w_codes, w_sf = self._weight_operand(f"mlp_linear_{layer_idx}_{i}", layer)
            act = None
            if i + 1 < len(layers):
                nxt = layers[i + 1]
                act = _ACT_MODULES.get(type(nxt))
                if isinstance(nxt, nn.GELU) and getattr(nxt, "approximate", "none") != "none":
                    act = None                            # the epilogue's GELU is the exact one
            feeds_linear = (act is not None and i + 2 < len(layers) and isinstance(layers[i + 2], nn.Linear)
                            and layers[i + 2].in_features % 32 == 0 and layers[i + 2].out_features % 32 == 0)
            if feeds_linear:
                # Linear -> activation -> Linear: the hidden activation leaves the first GEMM already quantised
                _, codes, sf = nv.gemm_fused(codes, sf, w_codes, w_sf, bias=bf16(layer.bias), activation=act,
                                             quantize_out=True, write_d=False)
                h = None
                i += 2
            elif act is not None:
                h, _, _ = nv.gemm_fused(codes, sf, w_codes, w_sf, bias=bf16(layer.bias), activation=act, quantize_out=False)
                codes = sf = None
                i += 2
            else:
                h = nv.gemm(codes, sf, w_codes, w_sf, bias=bf16(layer.bias))
                codes = sf = None
                i += 1
        return h.reshape(*lead, h.shape[-1]).to(out_dtype)
