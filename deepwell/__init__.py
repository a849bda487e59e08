"""Import-name alias: ``import deepwell`` resolves to the B200 implementation of the MXFP8 linear
path, so code written against the reference package (``deepwell.optimize``,
``deepwell.cutlass_kernels``, ``deepwell.kernels.cutlass_bindings``, ``deepwell.kernels.registry``)
runs unchanged.  Only the names of that path exist (of ``deepwell.engine`` only the MLP executor); the rest of the
reference package (capture, compile, probe, precision policy, attention) is not part of this build."""
import sys as _sys

import deepwell_b200 as _impl
from deepwell_b200 import DWLinear, DeepwellOptimizer, cutlass_kernels, kernels, optimize, optimize_for_blackwell  # noqa: F401
from deepwell_b200 import engine as _engine, optimizer as _optimizer
from deepwell_b200.kernels import blackwell_production as _bp, cutlass_bindings as _cb, production_kernels as _pk, registry as _reg

__version__ = _impl.__version__
for _name, _mod in (("cutlass_kernels", cutlass_kernels), ("kernels", kernels), ("optimizer", _optimizer),
                    ("kernels.cutlass_bindings", _cb), ("kernels.registry", _reg), ("kernels.production_kernels", _pk),
                    ("kernels.blackwell_production", _bp), ("engine", _engine)):
    _sys.modules[__name__ + "." + _name] = _mod
