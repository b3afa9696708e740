"""Host-side logic of the row-sharded pair track, on two CPU ranks (gloo): the all-to-all transpose of a row
shard, the row all-gather and the shard index arithmetic.  No GPU involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n: int, c: int):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kfold_b200 import sharded
        g = torch.Generator().manual_seed(7)
        z = torch.randn(n, n, c, generator=g)
        mask = torch.rand(n, n, generator=g) > 0.3
        r0, r1 = sharded.shard_rows(n, world, rank)
        assert r1 - r0 == n // world
        zt = sharded.transpose_shard(z[r0:r1].contiguous())
        assert torch.equal(zt, z.transpose(0, 1)[r0:r1])
        mt = sharded.transpose_shard(mask[r0:r1].to(torch.uint8).contiguous())
        assert torch.equal(mt.bool(), mask.t()[r0:r1])
        # transposing twice is the identity on the shard
        assert torch.equal(sharded.transpose_shard(zt), z[r0:r1])
        full = sharded.gather_rows(z[r0:r1].contiguous())
        assert torch.equal(full, z)
        # the gathered-operand layout the contraction consumes: rank after rank, each piece [channel][rows][n]
        piece = z[r0:r1].permute(2, 0, 1).contiguous()                       # [c][rows][n]
        gathered = sharded.gather_rows(piece).view(world, c, n // world, n)
        for q in range(world):
            q0, q1 = sharded.shard_rows(n, world, q)
            assert torch.equal(gathered[q], z[q0:q1].permute(2, 0, 1))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 8), (2, 12), (4, 16)])
def test_transpose_and_gather_on_cpu_ranks(world, n):
    mp.spawn(_worker, args=(world, _free_port(), n, 3), nprocs=world, join=True)


def test_shard_rows_rejects_uneven_split():
    from kfold_b200 import sharded
    with pytest.raises(ValueError):
        sharded.shard_rows(10, 4, 0)
    assert sharded.shard_rows(2048, 8, 3) == (768, 1024)
