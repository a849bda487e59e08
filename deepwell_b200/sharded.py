"""N-sharded (column-parallel) MXFP8 linear over torch.distributed — one process per GPU.

The reference has no distributed code (its ``autoplan`` returns a placeholder dict,
src/deepwell/__init__.py:45-83).  The linear path shards naturally along N:

    Y[:, n0:n1] = X . W[n0:n1, :]^T

X is replicated, each rank owns ``N / world`` rows of W, quantises them locally (scale blocks
run along K, so no block straddles ranks) and runs the same GEMM kernel on its shard.  No
collective is on the data path of the forward GEMM.  A collective appears only where the
consumer needs it:

    gather_output=True   all-gather of Y along N (NCCL over NVLink)
    backward             dX is a partial sum over the N shards -> all-reduce;
                         dW[n0:n1] is local.

The arithmetic is delegated to ``linear_fn`` (default: the native DWLinear function) so the
sharding logic itself can be exercised on CPU ranks (gloo) with a stand-in.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def shard_bounds(n: int, world: int, rank: int, multiple: int = 32) -> Tuple[int, int]:
    """Rows [n0, n1) of an N-row weight owned by `rank`: equal shards in units of `multiple`
    rows (the MX block, so dgrad's scale blocks along N never straddle ranks); the last
    ranks get one unit less when the units do not divide evenly."""
    if n % multiple:
        raise ValueError(f"N={n} is not a multiple of {multiple}")
    units = n // multiple
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return start * multiple, (start + count) * multiple


class _AllReduceGrad(torch.autograd.Function):
    """Identity in forward; all-reduce(sum) of the gradient in backward (dX partial sums)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _GatherColumns(torch.autograd.Function):
    """All-gather of [M, n_local] shards along N; backward keeps this rank's columns."""

    @staticmethod
    def forward(ctx, y, group, sizes, rank):
        world = len(sizes)
        ctx.sizes, ctx.rank = sizes, rank
        y = y.contiguous()
        widest = max(sizes)
        if y.shape[1] != widest:                      # uneven shards: pad to the widest, trim after
            y = torch.nn.functional.pad(y, (0, widest - y.shape[1]))
        flat = torch.empty((world * y.shape[0], widest), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(flat, y, group=group)      # rank-major concatenation along dim 0
        buf = flat.view(world, y.shape[0], widest)
        if len(set(sizes)) == 1:
            return buf.permute(1, 0, 2).reshape(y.shape[0], -1)
        return torch.cat([buf[r, :, :s] for r, s in enumerate(sizes)], dim=1)

    @staticmethod
    def backward(ctx, g):
        start = sum(ctx.sizes[: ctx.rank])
        return g[:, start:start + ctx.sizes[ctx.rank]].contiguous(), None, None, None


class ColumnParallelDWLinear(nn.Module):
    """DWLinear whose weight is split along N across the ranks of `group`."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = False,
                 group: Optional[dist.ProcessGroup] = None, device=None, dtype=None,
                 linear_fn: Optional[Callable] = None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features, self.out_features = in_features, out_features
        self.gather_output = gather_output
        self.sizes = [b - a for a, b in (shard_bounds(out_features, self.world, r) for r in range(self.world))]
        self.n0, self.n1 = shard_bounds(out_features, self.world, self.rank)
        n_local = self.n1 - self.n0
        if linear_fn is None:
            from .linear import DWLinear
            self.local = DWLinear(in_features, n_local, bias=bias, device=device, dtype=dtype)
            self._fn = None
        else:                           # CPU stand-in for tests of the sharding logic
            self.local = nn.Linear(in_features, n_local, bias=bias, device=device, dtype=dtype)
            self._fn = linear_fn

    @torch.no_grad()
    def load_full_weight(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """Copies this rank's rows of a full [N, K] weight (and [N] bias)."""
        self.local.weight.copy_(weight[self.n0:self.n1])
        if bias is not None and self.local.bias is not None:
            self.local.bias.copy_(bias[self.n0:self.n1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features)
        if self.world > 1 and x2d.requires_grad:
            x2d = _AllReduceGrad.apply(x2d, self.group)
        y = self.local(x2d) if self._fn is None else self._fn(x2d, self.local.weight, self.local.bias)
        if self.gather_output and self.world > 1:
            y = _GatherColumns.apply(y, self.group, self.sizes, self.rank)
        return y.reshape(*lead, y.shape[-1])
