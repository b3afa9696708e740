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
        assert torch.equal(sharded.transpose_shard(zt, add_to=z[r0:r1]), 2 * z[r0:r1])
        full = sharded.gather_rows(z[r0:r1].contiguous())
        assert torch.equal(full, z)
        # the gathered-operand layout the contraction consumes: rank after rank, each piece [channel][rows][n]
        piece = z[r0:r1].permute(2, 0, 1).contiguous()                       # [c][rows][n]
        gathered = sharded.gather_rows(piece).view(world, c, n // world, n)
        for q in range(world):
            q0, q1 = sharded.shard_rows(n, world, q)
            assert torch.equal(gathered[q], z[q0:q1].permute(2, 0, 1))
        # per-head rows gathered with one collective: (H, rows, n) -> (H, N, n)
        heads = z.permute(2, 0, 1)                                             # [c][n][n] stands in for [H][N][N]
        assert torch.equal(sharded.gather_head_rows(heads[:, r0:r1].contiguous()), heads)
        # the transposed mask is exchanged once per mask tensor and reused
        ops = sharded.ShardedPairOps()
        m_loc = mask[r0:r1].contiguous()
        mt1 = ops._transposed_mask(m_loc)
        assert torch.equal(mt1.bool(), mask.t()[r0:r1])
        assert ops._transposed_mask(m_loc) is mt1
        m_loc[0, 0] = ~m_loc[0, 0]                                             # an in-place edit invalidates the cache
        assert ops._transposed_mask(m_loc) is not mt1
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


def _worker_channel_sharded(rank: int, world: int, port: int, n: int, c: int):
    """The channel-sharded triangle contraction, with torch standing in for the kernels: operand channels written in
    packing.channel_shard_order, all-to-all, per-channel contraction read through the strides the kernel uses,
    all-to-all back; the result must be the row shard of the full einsum."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kfold_b200 import packing, sharded
        g = torch.Generator().manual_seed(11)
        a = torch.randn(c, n, n, generator=g)          # a[ch][i][k]
        b = torch.randn(c, n, n, generator=g)          # b[ch][j][k]
        t_full = torch.einsum("cik,cjk->cij", a, b)
        r0, r1 = sharded.shard_rows(n, world, rank)
        rows, cl = r1 - r0, c // world
        # what kfb_trimul_project writes with the permuted weights: [2c in shard order][rows][n] = [q][a, b][cl][rows][n]
        ab_nat = torch.cat([a[:, r0:r1], b[:, r0:r1]], dim=0)                 # natural order [a | b]
        order = packing.channel_shard_order(c, world)
        send = ab_nat[order].contiguous().view(world, 2, cl, rows, n)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        # kfb_trimul_contract_cs: rows (q, r) of a / b for this rank's channels, result laid out [q][cl][rows][n]
        a_cs = recv[:, 0].permute(1, 0, 2, 3).reshape(cl, n, n)
        b_cs = recv[:, 1].permute(1, 0, 2, 3).reshape(cl, n, n)
        assert torch.equal(a_cs, a[rank * cl:(rank + 1) * cl]) and torch.equal(b_cs, b[rank * cl:(rank + 1) * cl])
        t_cs = torch.einsum("cik,cjk->cij", a_cs, b_cs)                       # [cl][N][N]
        t_send = t_cs.view(cl, world, rows, n).permute(1, 0, 2, 3).contiguous()
        t_recv = torch.empty_like(t_send)
        dist.all_to_all_single(t_recv, t_send)
        t_loc = t_recv.view(c, rows, n)                                       # channel-major rows of this rank
        assert torch.allclose(t_loc, t_full[:, r0:r1], atol=1e-5)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,c", [(2, 8, 4), (4, 16, 8)])
def test_channel_sharded_contraction_algebra(world, n, c):
    mp.spawn(_worker_channel_sharded, args=(world, _free_port(), n, c), nprocs=world, join=True)


def test_channel_shard_order_is_a_permutation():
    from kfold_b200 import packing
    o = packing.channel_shard_order(128, 8)
    assert sorted(o.tolist()) == list(range(256))
    assert o[:3].tolist() == [0, 1, 2] and o[16] == 128 and o[32] == 16     # rank 0: a[0:16], b[0:16]; rank 1: a[16:32]


@pytest.mark.parametrize("c,world,parts", [(128, 8, 2), (128, 2, 2), (256, 4, 2), (64, 4, 1)])
def test_channel_shard_order_groups(c, world, parts):
    """The operand channel order of the grouped channel exchange: group h, rank q holds a- and b-channels
    h*(c/parts) + q*cl .. + cl, so that the results returned group by group and rank by rank are in channel order."""
    from kfold_b200 import packing
    cl = c // (world * parts)
    order = packing.channel_shard_order(c, world, parts).view(parts, world, 2, cl)
    assert sorted(order.reshape(-1).tolist()) == list(range(2 * c))
    for h in range(parts):
        for q in range(world):
            want = h * (c // parts) + q * cl + torch.arange(cl)
            assert torch.equal(order[h, q, 0], want) and torch.equal(order[h, q, 1], c + want)
    # the contraction results come back as [h][q][cl]: flat position = channel index
    back = order[:, :, 0].reshape(-1)
    assert torch.equal(back, torch.arange(c))
