"""Column-sharded compressed linear over NCCL (needs two GPUs; skipped on a single-GPU box)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dense(device):
    g = torch.Generator().manual_seed(11)
    layer = torch.nn.Linear(1024, 768, bias=True, dtype=torch.bfloat16)
    with torch.no_grad():
        layer.weight.copy_((torch.randn(768, 1024, generator=g) * 0.02).to(torch.bfloat16))
        layer.bias.copy_(torch.randn(768, generator=g).to(torch.bfloat16))
    x = torch.randn(304, 1024, generator=g).to(torch.bfloat16)
    return layer.to(device), x.to(device)


def _worker(rank: int, world: int, port: int, results):
    import entropack_b200 as ep
    from entropack_b200 import sharding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        dense, x = _dense(device)
        layer = sharding.ColumnShardedLinear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0), exchange="gather")
        out = layer(x)
        torch.cuda.synchronize()
        # the same layer with the exchange folded into the product's epilogue (peer stores + bounded barrier), three
        # forwards in a row so that both of its alternating output buffers and a reused one are read
        fused = sharding.ColumnShardedLinear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0), exchange="auto")
        scattered = [fused(x).clone() for _ in range(3)]
        fused.check()
        torch.cuda.synchronize()
        results[f"scatter{rank}"] = (fused.scatter_unavailable, [bool(torch.equal(s.view(torch.int16), out.view(torch.int16))) for s in scattered])
        # what a single device computes for the same two row shards, each compressed on its own
        pieces = []
        for r in range(world):
            rows = sharding.row_slice(dense.out_features, r, world)
            shard = torch.nn.Linear(1024, rows.end - rows.begin, bias=True, device=device, dtype=torch.bfloat16)
            with torch.no_grad():
                shard.weight.copy_(dense.weight[rows.begin : rows.end])
                shard.bias.copy_(dense.bias[rows.begin : rows.end])
            pieces.append(ep.CompressedLinear.from_linear(shard, config=ep.EntroPackLossyConfig(target_bpp=4.0))(x))
        expected = torch.cat(pieces, dim=-1)
        results[rank] = (tuple(out.shape), bool(torch.equal(out.view(torch.int16), expected.view(torch.int16))),
                         float((out.float() - dense(x).float()).norm() / dense(x).float().norm()))
    finally:
        dist.destroy_process_group()


def test_column_sharded_linear_all_gathers_outputs():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        shape, identical, relative = results[rank]
        assert shape == (304, 768) and identical and relative < 0.12
        unavailable, same = results[f"scatter{rank}"]
        assert unavailable is None, f"the scattered exchange fell back to the all-gather: {unavailable}"
        assert same == [True, True, True]


def test_one_process_can_drive_the_product_on_two_devices():
    """Kernel attributes (the dynamic shared memory limit) are per device: a process that multiplies on cuda:0 and then
    on cuda:1 must get the large-tile kernels on both."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from entropack_b200.linear import linear_forward

    generator = torch.Generator().manual_seed(3)
    x = torch.randn(2048, 1024, generator=generator).to(torch.bfloat16)
    w = (torch.randn(4608, 1024, generator=generator) * 0.02).to(torch.bfloat16)
    expected = x.float() @ w.float().t()
    for index in (0, 1):
        device = torch.device("cuda", index)
        with torch.cuda.device(device):
            out = linear_forward(x.to(device), w.to(device))
            torch.cuda.synchronize(device)
        assert float((out.float().cpu() - expected).abs().max() / expected.abs().max()) <= 1e-2
