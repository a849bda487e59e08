"""N-sharded (column-parallel) and K-sharded (row-parallel) MXFP8 linear over torch.distributed — one process per GPU.

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

A layer whose input arrives already split along its features (the output of a column-parallel
layer that was not gathered) is sharded along K instead (RowParallelDWLinear):

    Y = sum over ranks of X[:, k0:k1] . W[:, k0:k1]^T

Every rank quantises only its own K slice of X and W (scale blocks of 32 along K: the slices are
cut in units of 32, so no block straddles ranks), the partial products are summed by an
all-reduce, or by a reduce-scatter over the token rows when the consumer works on a slice of
the tokens.  A column-parallel layer followed by a row-parallel one (gate/up -> down of an MLP)
needs no collective between them and no rank quantises an activation it does not own.

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
    """All-gather of [M, n_local] shards along N; backward keeps this rank's columns.

    A collective library delivers every rank's shard as one contiguous block, so the gathered data is
    rank-major, [world, M, n_local].  ``blocked=True`` returns exactly that (no further pass over the data;
    for a consumer that addresses the columns as (rank, column) itself).  Otherwise the blocks are copied once
    into the column slices of the [M, N] result: one strided copy, the minimum a row-major result costs after
    such a collective."""

    @staticmethod
    def forward(ctx, y, group, sizes, rank, blocked):
        world = len(sizes)
        ctx.sizes, ctx.rank, ctx.blocked = sizes, rank, blocked
        y = y.contiguous()
        m, widest = y.shape[0], max(sizes)
        if y.shape[1] != widest:                      # uneven shards: pad to the widest, trim after
            y = torch.nn.functional.pad(y, (0, widest - y.shape[1]))
        buf = torch.empty((world, m, widest), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(buf.view(world * m, widest), y, group=group)      # rank-major
        if blocked:
            if len(set(sizes)) != 1:
                raise RuntimeError("the blocked layout needs equal shards")
            return buf
        out = torch.empty((m, sum(sizes)), dtype=y.dtype, device=y.device)
        start = 0
        for r, s in enumerate(sizes):
            out[:, start:start + s].copy_(buf[r, :, :s])
            start += s
        return out

    @staticmethod
    def backward(ctx, g):
        if ctx.blocked:
            return g[ctx.rank].contiguous(), None, None, None, None
        start = sum(ctx.sizes[: ctx.rank])
        return g[:, start:start + ctx.sizes[ctx.rank]].contiguous(), None, None, None, None


class _ReduceSum(torch.autograd.Function):
    """All-reduce(sum) of the partial products in forward; identity in backward (dY is replicated)."""

    @staticmethod
    def forward(ctx, y, group):
        y = y.contiguous().clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ReduceScatterRows(torch.autograd.Function):
    """Reduce-scatter(sum) of [M, N] partial products over the token rows: rank r keeps rows
    [r M / world, (r + 1) M / world).  Backward all-gathers the row slices of dY."""

    @staticmethod
    def forward(ctx, y, group, world):
        ctx.group, ctx.world = group, world
        y = y.contiguous()
        if y.shape[0] % world:
            raise RuntimeError(f"reduce-scatter over {world} ranks needs a token count divisible by it, got {y.shape[0]}")
        out = torch.empty((y.shape[0] // world, y.shape[1]), dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        full = torch.empty((g.shape[0] * ctx.world, g.shape[1]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(full, g, group=ctx.group)
        return full, None, None


class ColumnParallelDWLinear(nn.Module):
    """DWLinear whose weight is split along N across the ranks of `group`."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = False,
                 group: Optional[dist.ProcessGroup] = None, device=None, dtype=None,
                 linear_fn: Optional[Callable] = None, blocked_output: bool = False):
        """gather_output: all-gather Y along N.  blocked_output: return the gathered Y as [world, ..., n_local]
        (what the collective delivers) instead of copying it into [..., N]."""
        super().__init__()
        self.group = group
        self.blocked_output = blocked_output
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
            y = _GatherColumns.apply(y, self.group, self.sizes, self.rank, self.blocked_output)
            if self.blocked_output:
                return y.reshape(self.world, *lead, y.shape[-1])
        return y.reshape(*lead, y.shape[-1])


class RowParallelDWLinear(nn.Module):
    """DWLinear whose weight is split along K (its input features) across the ranks of `group`.

    input_is_parallel=True: x is this rank's feature slice [..., k1 - k0] (what an ungathered
    ColumnParallelDWLinear with the same world returns); False: x is the full [..., K] and the slice is taken here.
    scatter_output=False: the partial products are all-reduced, every rank returns the full Y [..., N];
    True: they are reduce-scattered over the token rows, rank r returns rows [r M / world, (r + 1) M / world)
    of the flattened [M, N] result.  The bias is added once, after the reduction."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, input_is_parallel: bool = True,
                 scatter_output: bool = False, group: Optional[dist.ProcessGroup] = None, device=None, dtype=None,
                 linear_fn: Optional[Callable] = None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features, self.out_features = in_features, out_features
        self.input_is_parallel, self.scatter_output = input_is_parallel, scatter_output
        self.k0, self.k1 = shard_bounds(in_features, self.world, self.rank)
        k_local = self.k1 - self.k0
        if linear_fn is None:
            from .linear import DWLinear
            self.local = DWLinear(k_local, out_features, bias=False, device=device, dtype=dtype)
            self._fn = None
        else:
            self.local = nn.Linear(k_local, out_features, bias=False, device=device, dtype=dtype)
            self._fn = linear_fn
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None

    @torch.no_grad()
    def load_full_weight(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """Copies this rank's columns of a full [N, K] weight (and the whole [N] bias)."""
        self.local.weight.copy_(weight[:, self.k0:self.k1])
        if bias is not None and self.bias is not None:
            self.bias.copy_(bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel:
            x = x[..., self.k0:self.k1]
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.k1 - self.k0)
        y = self.local(x2d) if self._fn is None else self._fn(x2d, self.local.weight, None)
        if self.world > 1:
            y = _ReduceScatterRows.apply(y, self.group, self.world) if self.scatter_output else _ReduceSum.apply(y, self.group)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if self.scatter_output and self.world > 1:
            return y                                   # [M / world, N]: a slice of the flattened token rows
        return y.reshape(*lead, self.out_features)
