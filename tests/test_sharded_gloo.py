"""World-size-2 CPU (gloo) test of the N-sharded linear: the sharding, gather and gradient
reduction logic with a plain matmul standing in for the GPU kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, gather):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deepwell_b200.sharded import ColumnParallelDWLinear
        torch.manual_seed(0)                         # same "replicated" tensors on every rank
        n, k, m = 160, 64, 24                        # 5 units of 32 rows: shards of 96 and 64 (uneven)
        w_full, b_full = torch.randn(n, k), torch.randn(n)
        x = torch.randn(2, m // 2, k, requires_grad=True)
        gy = torch.randn(2, m // 2, n)               # drawn before the shard-sized inits desynchronise the RNG
        layer = ColumnParallelDWLinear(k, n, bias=True, gather_output=gather, linear_fn=F.linear)
        layer.load_full_weight(w_full, b_full)
        assert layer.sizes == [96, 64]
        y = layer(x)
        ref = F.linear(x.detach(), w_full, b_full)
        n0, n1 = layer.n0, layer.n1
        if gather:
            assert y.shape == (2, m // 2, n) and torch.allclose(y, ref, atol=1e-5)
            y.backward(gy)
            gy_local = gy[..., n0:n1]
        else:
            assert y.shape == (2, m // 2, n1 - n0) and torch.allclose(y, ref[..., n0:n1], atol=1e-5)
            gy_local = gy[..., n0:n1]
            y.backward(gy_local)
        # dX is the sum over shards = the full-layer gradient; dW is local
        dx_ref = gy.reshape(-1, n) @ w_full
        assert torch.allclose(x.grad.reshape(-1, k), dx_ref, atol=1e-4)
        dw_ref = gy_local.reshape(-1, n1 - n0).t() @ x.detach().reshape(-1, k)
        assert torch.allclose(layer.local.weight.grad, dw_ref, atol=1e-4)
        assert torch.allclose(layer.local.bias.grad, gy_local.reshape(-1, n1 - n0).sum(0), atol=1e-4)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("gather", [False, True])
def test_column_parallel_world2(gather):
    mp.spawn(_worker, args=(2, _free_port(), gather), nprocs=2, join=True)


def _blocked_worker(rank, world, port):
    """gather_output with blocked_output=True: the rank-major [world, ..., n_local] result of the collective as it is."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deepwell_b200.sharded import ColumnParallelDWLinear
        torch.manual_seed(0)
        n, k, m = 128, 64, 12
        w_full = torch.randn(n, k)
        x = torch.randn(m, k, requires_grad=True)
        gy = torch.randn(world, m, n // world)
        layer = ColumnParallelDWLinear(k, n, bias=False, gather_output=True, blocked_output=True, linear_fn=F.linear)
        layer.load_full_weight(w_full)
        y = layer(x)
        ref = F.linear(x.detach(), w_full)
        assert y.shape == (world, m, n // world)
        for r in range(world):
            assert torch.allclose(y[r], ref[:, r * (n // world):(r + 1) * (n // world)], atol=1e-5)
        y.backward(gy)
        gy_full = torch.cat([gy[r] for r in range(world)], dim=1)
        assert torch.allclose(x.grad, gy_full @ w_full, atol=1e-4)
    finally:
        dist.destroy_process_group()


def test_column_parallel_blocked_gather_world2():
    mp.spawn(_blocked_worker, args=(2, _free_port()), nprocs=2, join=True)


def _row_worker(rank, world, port, scatter, parallel_input):
    """K-sharded layer: partial products summed by all-reduce or reduce-scatter over the token rows; every gradient
    against the unsharded layer."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deepwell_b200.sharded import RowParallelDWLinear
        torch.manual_seed(0)
        n, k, m = 96, 160, 24                        # 5 units of 32 columns: K slices of 96 and 64 (uneven)
        w_full, b_full = torch.randn(n, k), torch.randn(n)
        x_full = torch.randn(2, m // 2, k)
        gy = torch.randn(m, n)
        layer = RowParallelDWLinear(k, n, bias=True, input_is_parallel=parallel_input, scatter_output=scatter,
                                    linear_fn=F.linear)
        layer.load_full_weight(w_full, b_full)
        k0, k1 = layer.k0, layer.k1
        assert (k0, k1) == ((0, 96) if rank == 0 else (96, 160))
        x = (x_full[..., k0:k1] if parallel_input else x_full).clone().requires_grad_(True)
        y = layer(x)
        ref = F.linear(x_full, w_full, b_full).reshape(m, n)
        rows = slice(rank * m // world, (rank + 1) * m // world) if scatter else slice(0, m)
        assert y.reshape(-1, n).shape == ref[rows].shape
        assert torch.allclose(y.reshape(-1, n), ref[rows], atol=1e-4)
        y.reshape(-1, n).backward(gy[rows])
        dx_ref = (gy @ w_full).reshape(2, m // 2, k)           # every rank's dX uses the dY of ALL token rows
        got_dx = x.grad if parallel_input else x.grad[..., k0:k1]
        assert torch.allclose(got_dx, dx_ref[..., k0:k1], atol=1e-4)
        if not parallel_input:                                  # columns owned by the other rank get no gradient here
            other = torch.ones(k, dtype=torch.bool)
            other[k0:k1] = False
            assert x.grad[..., other].abs().max() == 0
        dw_ref = gy.t() @ x_full.reshape(m, k)
        assert torch.allclose(layer.local.weight.grad, dw_ref[:, k0:k1], atol=1e-4)
        assert torch.allclose(layer.bias.grad, gy[rows].sum(0), atol=1e-4)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scatter,parallel_input", [(False, True), (True, True), (False, False)])
def test_row_parallel_world2(scatter, parallel_input):
    mp.spawn(_row_worker, args=(2, _free_port(), scatter, parallel_input), nprocs=2, join=True)


def _mlp_worker(rank, world, port):
    """Column-parallel up-projection feeding a row-parallel down-projection with no collective between them."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deepwell_b200.sharded import ColumnParallelDWLinear, RowParallelDWLinear
        torch.manual_seed(0)
        h, f, m = 64, 256, 16
        w1, w2 = torch.randn(f, h) * 0.1, torch.randn(h, f) * 0.1
        x = torch.randn(m, h)
        up = ColumnParallelDWLinear(h, f, bias=False, gather_output=False, linear_fn=F.linear)
        down = RowParallelDWLinear(f, h, bias=False, input_is_parallel=True, linear_fn=F.linear)
        up.load_full_weight(w1)
        down.load_full_weight(w2)
        assert (up.n0, up.n1) == (down.k0, down.k1)
        y = down(torch.relu(up(x)))
        assert torch.allclose(y, F.linear(torch.relu(F.linear(x, w1)), w2), atol=1e-4)
    finally:
        dist.destroy_process_group()


def test_column_then_row_parallel_mlp_world2():
    mp.spawn(_mlp_worker, args=(2, _free_port()), nprocs=2, join=True)
