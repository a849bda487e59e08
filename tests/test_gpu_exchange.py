"""GPU tests of deepwell_b200.exchange on ONE GPU (a process group of one rank): the buffer handling, the batched
quantiser launches behind it and the pitched copy of the C ABI.  The traffic between GPUs is checked byte for byte inside
`bench.py --gpus N` (keys `exchange.parity`, `with_gather.copy_engines.parity_vs_nccl_all_gather`)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


@pytest.fixture(scope="module")
def nv(native_lib):
    from deepwell_b200 import _native
    assert torch.cuda.is_available(), "the parity tests need a GPU"
    assert native_lib.dw_mxfp8_device_supported(0) == 1, "sm_100a device required"
    return _native


@pytest.fixture(scope="module")
def one_rank_group():
    created = False
    if not dist.is_initialized():
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        created = True
    yield
    if created:
        dist.destroy_process_group()


def test_pitched_copy_places_a_block_of_columns(nv):
    g = torch.Generator(device="cuda").manual_seed(5)
    src = torch.randn(300, 96, device="cuda", generator=g).bfloat16()
    dst = torch.zeros(300, 512, dtype=torch.bfloat16, device="cuda")
    nv.copy_2d_async(dst.data_ptr() + 128 * 2, 512 * 2, src.data_ptr(), 96 * 2, 96 * 2, 300, dst.device)
    torch.cuda.synchronize()
    assert torch.equal(dst[:, 128:224], src) and not bool(dst[:, :128].any()) and not bool(dst[:, 224:].any())
    L = nv.load()
    assert L.dw_mxfp8_copy_2d_async(dst.data_ptr(), 8, src.data_ptr(), 192, 192, 4, None) == -1     # pitch shorter than the row
    assert L.dw_mxfp8_copy_2d_async(None, 0, None, 0, 0, 0, None) == 0                              # nothing to copy


@pytest.mark.parametrize("shared", [None, [128, 0], [0, 384]])
def test_exchange_of_one_rank_is_the_plain_quantisation(nv, one_rank_group, shared):
    from deepwell_b200.exchange import QuantizedRowExchange
    g = torch.Generator(device="cuda").manual_seed(11)
    xs = [(torch.randn(256, 512, device="cuda", generator=g) * 0.5).bfloat16(),
          (torch.randn(384, 128, device="cuda", generator=g) * 3.0).bfloat16()]
    w = (torch.randn(128, 256, device="cuda", generator=g) * 0.02).bfloat16()
    wc = torch.empty(128, 256, dtype=torch.uint8, device="cuda")
    ws = torch.empty(nv.scale_bytes(128, 256, nv.SF_TILED), dtype=torch.uint8, device="cuda")
    ex = QuantizedRowExchange([tuple(x.shape) for x in xs])
    ex.set_shared_rows(shared)
    for slot in (0, 1):
        launches = ex.quantise_and_push(xs, slot, extra=[(w, wc, ws)])
        ex.fence(slot)
        assert launches == 1                                    # every piece and the extra operand in one launch
        for i, x in enumerate(xs):
            codes, scales = ex.operand(slot, i)
            ec, es = nv.quantize(x, nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
            assert torch.equal(codes, ec.view(torch.uint8)) and torch.equal(scales, es.view(torch.uint8).reshape(-1))
        ec, es = nv.quantize(w, nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED)
        assert torch.equal(wc, ec.view(torch.uint8)) and torch.equal(ws, es.view(torch.uint8).reshape(-1))
    with pytest.raises(ValueError):
        ex.set_shared_rows([100, 0])
    with pytest.raises(ValueError):
        QuantizedRowExchange([(200, 64)])


@pytest.mark.parametrize("layout", ["blocked", "row_major"])
def test_column_gather_of_one_rank(nv, one_rank_group, layout):
    from deepwell_b200.exchange import ColumnGather
    g = torch.Generator(device="cuda").manual_seed(13)
    ys = [torch.randn(256, 64, device="cuda", generator=g).bfloat16(), torch.randn(130, 24, device="cuda", generator=g).bfloat16()]
    cg = ColumnGather([tuple(y.shape) for y in ys], layout=layout, slots=2)
    for slot in (0, 1):
        for i, y in enumerate(ys):
            cg.shard(i, slot).copy_(y * (slot + 1))
            cg.push(i, slot)
    cg.fence()
    torch.cuda.synchronize()
    for slot in (0, 1):
        for i, y in enumerate(ys):
            full = cg.full(i, slot)
            assert torch.equal(full[0] if layout == "blocked" else full, y * (slot + 1))
    with pytest.raises(ValueError):
        ColumnGather([(64, 12)], layout=layout)
