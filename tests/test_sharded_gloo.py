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
