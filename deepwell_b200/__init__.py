"""deepwell_b200 — B200 (sm_100a) implementation of Deepwell's MXFP8 linear path.

Public surface (names of the reference package ``deepwell``):
    optimize, DeepwellOptimizer        src/deepwell/optimizer.py
    DWLinear                           the module the reference's optimizer leaves as a TODO
    cutlass_kernels                    the extension-module API (csrc/python_bindings.cpp)
    kernels.cutlass_bindings, kernels.registry
    engine.ExecutableModel             its MLP executor (_mlp_with_cutlass, src/deepwell/engine.py:132-209)
    sharded                            N-sharded (column-parallel) and K-sharded (row-parallel) linear over torch.distributed
"""
__version__ = "0.1.0"

from .optimizer import DeepwellOptimizer, optimize          # noqa: E402
from .linear import DWLinear                                # noqa: E402
from . import cutlass_kernels, kernels                      # noqa: E402
from .kernels.production_kernels import optimize_for_blackwell   # noqa: E402

__all__ = ["optimize", "optimize_for_blackwell", "DeepwellOptimizer", "DWLinear", "cutlass_kernels", "kernels", "__version__"]
