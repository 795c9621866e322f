"""Tensor-parallel block on two GPUs (NCCL) against the single-rank oracle.  Skipped when fewer
than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import inputs, layers
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from energonai_b200 import tp
        from energonai_b200.model import Block1D
        from energonai_b200.sharding import shard_block_state
        tp.init_tp(world)
        h, H, f, B, S = 512, 8, 2048, 3, 40
        gen = torch.Generator().manual_seed(9)
        bp = inputs.block_params(gen, h, f, rich=True, std=0.04)
        x = torch.randn(B, S + 2, h, generator=gen)
        mask = torch.ones(B, S)
        mask[2, :11] = 0
        ok = True
        for fused in (False, True):
            blk = Block1D(h, H, f / h, activation=torch.nn.functional.relu, dtype=torch.float16, fused_qkv=fused).cuda()
            full = {k: v.half() for k, v in layers.block_to_reference_state(bp, fused).items()}
            blk.load_state_dict(shard_block_state(full, rank, world))
            ref = layers.OracleBlock(bp, H, "relu")
            with torch.inference_mode():
                for step in range(3):
                    cur = S + step
                    m = torch.cat([mask, torch.ones(B, step)], 1)
                    m4 = (1.0 - m.view(B, 1, 1, cur)) * -10000.0
                    out = blk(x[:, :cur].half().cuda(), m4.half().cuda(), first_cache=(step == 0)).float().cpu()
                    exp = ref(x[:, :cur], m4, step == 0)
                    a, b = (out[m.bool()], exp[m.bool()]) if step == 0 else (out[:, -1], exp[:, -1])
                    ok = ok and bool(((a - b).abs() <= 2e-2 + 1e-2 * b.abs()).all())
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_block_matches_oracle():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
