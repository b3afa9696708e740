"""Row-sharded Pairformer block on 2 GPUs against the single-GPU block (needs >= 2 CUDA devices)."""
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


def _worker(rank: int, world: int, port: int, n: int, exchange: str, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from kfold_b200 import sharded
    sharded.apply_nccl_env_defaults()
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from kfold_b200 import _lib as L
        from kfold_b200 import modules as M
        import synth
        w = synth.pairformer_block_weights(21)
        z, pm, m = synth.pair_inputs(21, n, 128, 1, pad_frac=0.1)
        s = synth.single_inputs(21, n, 384, 1)
        blk = M.PairformerBlock().to(dev)
        blk.load_state_dict(w, strict=True)
        zb, sb = z.to(dev, torch.bfloat16), s.to(dev, torch.bfloat16)
        with torch.no_grad():
            z_ref, s_ref = blk(zb.clone(), sb.clone(), pm.to(dev), m.to(dev))
            r0, r1 = sharded.shard_rows(n, world, rank)
            sblk = sharded.ShardedPairformerBlock(blk, exchange=exchange)
            z_loc, s_out = sblk(zb[0, r0:r1].contiguous(), sb.clone(), pm[0, r0:r1].to(dev).contiguous(), m.to(dev))
        torch.cuda.synchronize()
        status = L.device_status()
        ref = z_ref[0, r0:r1].float()
        ez = float((z_loc.float() - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())
        es = float((s_out.float() - s_ref.float()).pow(2).mean().sqrt() / s_ref.float().pow(2).mean().sqrt())
        exact = bool(torch.equal(z_loc, z_ref[0, r0:r1]))
        q.put((rank, status, ez, es, exact))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["gather", "channel"])
@pytest.mark.parametrize("n", [128, 256, 384])
def test_sharded_block_matches_single_gpu(n, exchange):
    """Both exchanges of the triangle multiplication: the all-gather of b and the channel-sharded all-to-all."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    mp.spawn(_worker, args=(world, _free_port(), n, exchange, q), nprocs=world, join=True)
    results = [q.get(timeout=10) for _ in range(world)]
    for rank, status, ez, es, exact in results:
        assert status == 0
        # same kernels and operands; the ending-node update is rounded to bf16 once more before it is added (it travels
            # through the all-to-all), hence a few 1e-3 of RMS rather than bit equality
        assert ez < 6e-3 and es < 6e-3, f"rank {rank}: z {ez:.3e} s {es:.3e} (bit-exact: {exact})"
