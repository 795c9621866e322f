"""Host-side tensor-parallel logic on CPU with two gloo ranks: the weight-sharding helper and
the TP context's all-reduce reproduce the single-rank layer output when each rank evaluates
its shard (with the oracle's math standing in for the CUDA kernels, which need a GPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from oracle import inputs, layers


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fused, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from energonai_b200 import tp as tpmod
        from energonai_b200.sharding import shard_block_state
        ctx = tpmod.init_tp(world)
        assert (ctx.rank, ctx.world_size) == (rank, world)
        h, H, f = 128, 4, 512
        gen = torch.Generator().manual_seed(3)
        bp = inputs.block_params(gen, h, f, rich=True, std=0.08)
        x = torch.randn(2, 6, h, generator=gen)
        shard = shard_block_state(layers.block_to_reference_state(bp, fused), rank, world)
        hl, d = h // world, h // H
        if fused:
            k_w, v_w, q_w = shard["attn.query_key_value.weight"].split(hl, 0)
            k_b, v_b, q_b = shard["attn.query_key_value.bias"].split(hl, 0)
        else:
            q_w, k_w, v_w = (shard[f"attn.{n}.weight"] for n in ("query_", "key_", "value_"))
            q_b, k_b, v_b = (shard[f"attn.{n}.bias"] for n in ("query_", "key_", "value_"))
        n1 = F.layer_norm(x, (h,), shard["norm1.module.weight"], shard["norm1.module.bias"])
        q, k, v = (F.linear(n1, w, b).view(2, 6, H // world, d).permute(0, 2, 1, 3)
                   for w, b in ((q_w, q_b), (k_w, k_b), (v_w, v_b)))
        s = (q * d ** -0.5) @ k.transpose(-1, -2)
        s = torch.where(torch.tril(torch.ones(6, 6, dtype=torch.bool)), s, torch.tensor(-1e4))
        ctxv = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(2, 6, hl)
        part = F.linear(ctxv, shard["attn.dense.weight"])
        if rank == 0:                                   # bias and residual enter the sum once
            part = part + shard["attn.dense.bias"] + x
        x1 = ctx.all_reduce(part)
        n2 = F.layer_norm(x1, (h,), shard["norm2.module.weight"], shard["norm2.module.bias"])
        part = F.linear(torch.relu(F.linear(n2, shard["mlp.dense_1.weight"], shard["mlp.dense_1.bias"])),
                        shard["mlp.dense_2.weight"])
        if rank == 0:
            part = part + shard["mlp.dense_2.bias"] + x1
        out = ctx.all_reduce(part)
        ref = layers.OracleBlock(bp, H, "relu")(x, None, True)
        ok = torch.allclose(out, ref, atol=2e-5, rtol=1e-5)
        gathered = ctx.all_gather_last_dim(torch.full((2, 3), float(rank)))
        ok = ok and gathered.shape == (2, 3 * world) and gathered[0, -1].item() == world - 1
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused", [False, True])
def test_two_rank_block_matches_single_rank(fused):
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, fused, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_default_context_is_single_rank():
    from energonai_b200 import tp as tpmod
    ctx = tpmod.set_tp(None)
    t = torch.ones(3)
    assert ctx.world_size == 1 and ctx.all_reduce(t) is t
    with pytest.raises(ValueError):
        tpmod.divide(10, 4)


def _vocab_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from energonai_b200 import tp as tpmod
        from energonai_b200.nn import VocabParallelEmbedding1D
        from energonai_b200.sharding import shard_model_state
        ctx = tpmod.init_tp(world)
        V, h = 64, 16
        gen = torch.Generator().manual_seed(8)
        full = {"embed.word_embeddings.weight": torch.randn(V, h, generator=gen),
                "embed.position_embeddings.weight": torch.randn(10, h, generator=gen),
                "head.dense.weight": torch.randn(V, h, generator=gen), "norm.module.weight": torch.ones(h)}
        shard = shard_model_state(full, rank, world, vocab_parallel=True)
        ok = shard["embed.word_embeddings.weight"].shape == (V // world, h) and shard["head.dense.weight"].shape == (V // world, h)
        ok = ok and shard["embed.position_embeddings.weight"].shape == (10, h)
        emb = VocabParallelEmbedding1D(V, h, padding_idx=0)
        with torch.no_grad():
            emb.weight.copy_(shard["embed.word_embeddings.weight"])
        ids = torch.randint(0, V, (3, 7), generator=gen)
        ok = ok and torch.equal(emb(ids), F.embedding(ids, full["embed.word_embeddings.weight"]))
        x = torch.randn(3, h, generator=gen)
        logits = ctx.all_gather_last_dim(F.linear(x, shard["head.dense.weight"]))
        ok = ok and torch.allclose(logits, F.linear(x, full["head.dense.weight"]), atol=1e-6)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_vocab_parallel_embedding_and_head_shards():
    """Vocabulary split over two ranks: masked local lookups summed by the all-reduce equal the
    full lookup, and the gathered per-rank logits equal the full projection."""
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_vocab_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
