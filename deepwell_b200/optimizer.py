"""``optimize()`` — module-tree rewrite that puts the MXFP8 path behind every nn.Linear.

Same entry point and keyword arguments as the reference (src/deepwell/optimizer.py:252-289)
and the same DeepwellOptimizer surface (stats dict :40-45, deep copy unless ``inplace``
:100-101, recursive replacement that does not descend into a replaced module :124-144).
The branch the reference leaves as a TODO (``nn.Linear`` with ``precision == "mxfp8"``,
:206-212) is the one implemented here.  The attention replacement of the reference
(:155-204) belongs to a different path and is not part of this package: attention modules
are left as they are (their inner nn.Linear projections are still visited).
"""
from __future__ import annotations

import copy
from typing import Dict, Optional, Sequence

import torch.nn as nn

from .linear import DWLinear


class DeepwellOptimizer:
    def __init__(self, precision: str = "bf16", target: str = "blackwell", verbose: bool = True, profile: bool = False,
                 policy=None, sensitive_layers: Optional[Sequence[str]] = None):
        """``policy``: a precision policy in the reference's shape (an object with ``config.sensitive_layers``,
        src/deepwell/precision/policy.py:102-109) or ``sensitive_layers``: substrings of qualified module names.
        A Linear whose lower-cased name contains one of them stays in its own precision, as
        PrecisionPolicy.assign_layer_precision decides (:138-151) — a policy the reference's optimize() never
        consults.  Default: none, every eligible Linear is replaced."""
        if sensitive_layers is None and policy is not None:
            sensitive_layers = getattr(getattr(policy, "config", policy), "sensitive_layers", None)
        self.sensitive_layers = [s.lower() for s in (sensitive_layers or [])]
        self.precision = precision
        self.target = target
        self.verbose = verbose
        self.profile = profile
        self.stats: Dict[str, int] = self._zero_stats()
        self.skipped = []          # (name, reason) of Linear layers left unreplaced

    @staticmethod
    def _zero_stats() -> Dict[str, int]:
        return {"modules_replaced": 0, "attention_modules": 0, "linear_modules": 0, "other_modules": 0}

    def optimize(self, model: nn.Module, inplace: bool = False) -> nn.Module:
        if self.verbose:
            bar = "=" * 60
            print(f"\n{bar}\nDeepwell Optimizer - {self.target.upper()} {self.precision.upper()}\n{bar}")
        if not inplace:
            model = copy.deepcopy(model)
        self.stats = self._zero_stats()
        self.skipped = []
        self._optimize_recursive(model)
        if self.profile:
            self._add_profiling_hooks(model)
        if self.verbose:
            self._print_summary()
        return model

    def _optimize_recursive(self, module: nn.Module, prefix: str = "") -> None:
        swaps = []
        for name, child in module.named_children():
            full = f"{prefix}.{name}" if prefix else name
            new = self._try_optimize_module(child, full)
            if new is None:
                self._optimize_recursive(child, full)
            else:
                swaps.append((name, new))
        for name, new in swaps:
            setattr(module, name, new)

    def _try_optimize_module(self, module: nn.Module, name: str) -> Optional[nn.Module]:
        if self.precision != "mxfp8" or type(module) is not nn.Linear:
            return None
        if any(s in name.lower() for s in self.sensitive_layers):
            self.skipped.append((name, "named sensitive by the precision policy"))
            if self.verbose:
                print(f"  [{name}] Linear kept in its own precision (sensitive layer)")
            return None
        if module.in_features % 32 or module.out_features % 32:
            self.skipped.append((name, "in/out features not multiples of the 32-element MX block"))
            if self.verbose:
                print(f"  [{name}] Linear kept (features not multiples of 32)")
            return None
        if self.verbose:
            print(f"  [{name}] Linear -> DWLinear")
        self.stats["modules_replaced"] += 1
        self.stats["linear_modules"] += 1
        return DWLinear.from_linear(module)

    def _add_profiling_hooks(self, model: nn.Module) -> None:
        """Counts forward calls per DWLinear in ``module.dw_calls`` (the reference registers a no-op, :216-229)."""
        def hook(mod, _inp, _out):
            mod.dw_calls = getattr(mod, "dw_calls", 0) + 1
        for m in model.modules():
            if isinstance(m, DWLinear):
                m.register_forward_hook(hook)

    def _print_summary(self) -> None:
        bar = "=" * 60
        print(f"\n{bar}\nOptimization Summary\n{bar}")
        print(f"Total modules replaced: {self.stats['modules_replaced']}")
        print(f"  - Attention modules:  {self.stats['attention_modules']}")
        print(f"  - Linear modules:     {self.stats['linear_modules']}")
        print(f"  - Other modules:      {self.stats['other_modules']}")
        print(bar)
        if self.stats["modules_replaced"]:
            print("\nLinear layers now run quantise + block-scaled GEMM in MXFP8 (forward, dgrad, wgrad).")
        else:
            print("\nNo optimizable modules found")


def optimize(model: nn.Module, precision: str = "bf16", target: str = "blackwell", verbose: bool = True,
             profile: bool = False, inplace: bool = False, policy=None,
             sensitive_layers: Optional[Sequence[str]] = None) -> nn.Module:
    """deepwell.optimize(model, precision="mxfp8"): every nn.Linear whose feature sizes are
    multiples of 32 becomes a DWLinear sharing the same parameters, except those a precision
    policy names sensitive (``policy`` / ``sensitive_layers``, see DeepwellOptimizer)."""
    return DeepwellOptimizer(precision=precision, target=target, verbose=verbose, profile=profile, policy=policy,
                             sensitive_layers=sensitive_layers).optimize(model, inplace=inplace)
