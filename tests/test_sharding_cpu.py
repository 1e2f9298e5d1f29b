"""Layer partitioning and the output all-gather on CPU (gloo, world size 2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from entropack_b200 import sharding


def test_dit_layer_list_has_276_linears():
    shapes = sharding.dit_layer_shapes()
    assert len(shapes) == 276
    assert set(shapes) == {(3840, 3840), (11520, 3840), (10240, 3840), (3840, 10240)}
    targets = sharding.mixed_bit_targets(shapes)
    weights = [r * c for r, c in shapes]
    mean = sum(t * w for t, w in zip(targets, weights)) / sum(weights)
    assert abs(mean - 2.3) < 0.01 and min(targets) > 1.0 and max(targets) < 4.5


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_is_complete_and_balanced(world):
    sizes = [r * c for r, c in sharding.dit_layer_shapes()]
    shares = sharding.partition_layers(sizes, world)
    assert sorted(i for share in shares for i in share) == list(range(len(sizes)))
    loads = [sum(sizes[i] for i in share) for share in shares]
    assert max(loads) - min(loads) <= max(sizes)
    assert shares == sharding.partition_layers(sizes, world)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank "compresses" only its share; the stand-in compressor records which layers it saw
        weights = [torch.full((4 + i, 8), float(i)) for i in range(7)]
        share = sharding.compress_layers(weights, None, compress_fn=lambda w, c: float(w.sum()))
        gathered = [None] * world
        dist.all_gather_object(gathered, share)
        merged = {k: v for part in gathered for k, v in part.items()}
        # column-sharded output gather
        full = torch.arange(6 * 8, dtype=torch.float32).reshape(6, 8)
        rows = sharding.row_slice(8, rank, world)
        out = sharding.gather_columns(full[:, rows.begin : rows.end].contiguous())
        results[rank] = (sorted(share), merged, torch.equal(out, full))
    finally:
        dist.destroy_process_group()


def test_two_ranks_share_layers_and_gather_outputs():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    shares = [results[r][0] for r in range(world)]
    assert sorted(shares[0] + shares[1]) == list(range(7)) and not set(shares[0]) & set(shares[1])
    for r in range(world):
        assert results[r][1] == {i: float((4 + i) * 8 * i) for i in range(7)}
        assert results[r][2]


def test_binding_near_a_gpu_is_a_no_op_without_one():
    """No NVML device here: the helper reports that it changed nothing and leaves the affinity as it was."""
    import os

    from entropack_b200 import sharding

    before = os.sched_getaffinity(0)
    assert sharding.bind_host_thread_near(0) is None
    assert os.sched_getaffinity(0) == before
