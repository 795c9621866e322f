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


def _mark(rank, what):
    """Progress line in the run's output folder (when that folder exists): shows how far a rank got if a run
    has to be ended from outside."""
    out = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpurun_out")
    if os.path.isdir(out):
        with open(os.path.join(out, f"tp_test_rank{rank}.log"), "a") as f:
            f.write(what + "\n")


def _leave(rank, ret, ok):
    """Ends a rank.  A rank that failed must not linger in collective teardown while its peer
    waits for it inside a collective: it reports and exits at once, which lets the spawner end
    the other rank too."""
    import sys
    import traceback
    import torch.distributed as dist
    _mark(rank, f"leaving ok={ok}")
    if ok:
        dist.destroy_process_group()
        _mark(rank, "process group destroyed")
        return
    traceback.print_exc()
    _mark(rank, traceback.format_exc())
    try:
        from energonai_b200 import tp
        from energonai_b200.gemm import device_status
        peer = tp.get_tp().peer
        print(f"rank {rank}: device status {device_status(clear=False)}, context status "
              f"{peer.status(clear=False) if peer is not None else None}", file=sys.stderr, flush=True)
    except Exception:                                            # noqa: BLE001
        pass
    ret[rank] = False
    sys.stderr.flush()
    os._exit(1)


def _worker(rank, world, port, ret, use_peer=False):
    import torch.distributed as dist
    from oracle import inputs, layers
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from energonai_b200 import tp
        from energonai_b200.model import Block1D
        from energonai_b200.sharding import shard_block_state
        ctx = tp.init_tp(world)
        h, H, f, B, S = 512, 8, 2048, 3, 40
        if use_peer:
            ctx.enable_peer_exchange(16, 5120, bulk_rows=512)
            assert ctx.peer is not None
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
        if use_peer:
            # the fused exchange against NCCL on the same operands: every rank gets the same bits
            from energonai_b200.gemm import gemm, device_status
            g = torch.Generator(device="cuda").manual_seed(100 + rank)
            for M, N, K in ((16, 512, 1024), (3, 2048, 256), (16, 5120, 640)):
                a = torch.randn(M, K, device="cuda", generator=g).half()
                w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).half()
                bias = torch.randn(N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)).half()
                for _ in range(3):                                    # consecutive calls alternate the buffers
                    fused = gemm(a, w, bias=bias, peer=ctx.peer)
                part = (a.float() @ w.float().t())
                dist.all_reduce(part)
                exp = part + bias.float()
                ok = ok and bool(((fused.float() - exp).abs() <= 2e-3 * exp.abs() + 2e-3 * exp.abs().max()).all())
                gathered = [torch.empty_like(fused) for _ in range(world)]
                dist.all_gather(gathered, fused)
                ok = ok and all(torch.equal(gathered[0], t) for t in gathered)
            ok = ok and device_status()[0] == 0
        ret[rank] = ok
    except BaseException:                                        # noqa: BLE001
        _leave(rank, ret, False)
    _leave(rank, ret, True)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("use_peer", [False, True])
def test_two_gpu_block_matches_oracle(use_peer):
    """use_peer=False: NCCL all-reduce after each row-parallel GEMM; use_peer=True: generation
    steps run the all-reduce inside the GEMM epilogue over NVLink peer stores."""
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret, use_peer), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _model_worker(rank, world, port, ret, use_peer=False):
    """A small OPT-shaped PipelineModel with vocab-parallel embedding and LM head on `world` GPUs
    against the same weights run on one rank.  use_peer: the generation steps run as chained
    launches that carry the all-reduces over NVLink peer memory (the library's own exchange)."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from energonai_b200 import tp
        from energonai_b200.model import PipelineModel
        from energonai_b200.sharding import shard_model_state
        kw = dict(vocab_size=1024, max_seq_len=128, hidden_size=256, num_heads=4, depth=2, mlp_ratio=4.0,
                  activation=torch.nn.functional.relu, dtype=torch.float16, fused_qkv=False, model_name="opt")
        tp.set_tp(None)                                      # single-rank context: the full model
        torch.manual_seed(21)
        full = PipelineModel(**kw).cuda().eval()
        with torch.no_grad():                               # livelier LayerNorms than the initial 1 / 0
            for name, p in full.named_parameters():
                if ".module." in name:
                    p.add_(0.1 * torch.randn_like(p))
        ids = torch.randint(3, 1024, (3, 11), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
        mask = torch.ones_like(ids)
        mask[1, :4] = 0
        record = {}
        want = full(input_ids=ids, attention_mask=mask, max_tokens=24, top_k=1, record=record)
        ctx = tp.init_tp(world)
        _mark(rank, f"model test use_peer={use_peer}: reference tokens done")
        if use_peer:
            ctx.enable_peer_exchange(16, 5120, bulk_rows=512)
            _mark(rank, "exchange enabled")
            # the stand-alone one-shot all-reduce against NCCL, several sizes and dtypes
            for dt, n in ((torch.float16, 4096), (torch.bfloat16, 1024 * 40), (torch.float32, 20)):
                t = (torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)) * 3).to(dt)
                want_t = t.float().clone()
                dist.all_reduce(want_t)
                for _ in range(3):
                    got_t = ctx.peer.all_reduce(t.clone())
                assert float((got_t.float() - want_t).abs().max()) <= 2e-2 * float(want_t.abs().max()) + 1e-6
                both = [torch.empty_like(got_t) for _ in range(world)]
                dist.all_gather(both, got_t)
                assert all(torch.equal(both[0], b) for b in both)      # bit-identical on every rank
                _mark(rank, f"one-shot all-reduce {dt} x {n} ok")
            bad = torch.tensor([float(ctx.peer.status(clear=False)[0] != 0)], device="cuda")
            dist.all_reduce(bad)                  # agree on the outcome before anybody may leave
            assert float(bad) == 0, f"rank {rank}: context status {ctx.peer.status()}"
        model = PipelineModel(vocab_parallel=True, **kw).cuda().eval()
        model.load_state_dict(shard_model_state(full.state_dict(), rank, world, vocab_parallel=True))
        assert model.embed.word_embeddings.weight.shape[0] == 1024 // world
        record_tp = {}
        _mark(rank, "sharded model built")
        got = model(input_ids=ids, attention_mask=mask, max_tokens=24, top_k=1, record=record_tp)
        _mark(rank, "eager generation done")
        if use_peer:
            from energonai_b200.gemm import device_status
            replayed = model(input_ids=ids, attention_mask=mask, max_tokens=24, top_k=1)      # captured step, fused exchange
            _mark(rank, "replayed generation done")
            assert model._decode_state["chain_mode"] is None and model._decode_state["graph"] is not None
            model.use_decode_chain = True                                                     # the chained form of the step
            model._decode_state = None
            chained = model(input_ids=ids, attention_mask=mask, max_tokens=24, top_k=1)
            _mark(rank, "chained generation done")
            assert model._decode_state["chain_mode"] == "exchange" and model._decode_state["graph"] is not None
            agree = torch.tensor([float((chained[:, 11:15] == want[:, 11:15]).float().mean())], device="cuda")
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            assert float(agree) >= 0.9
            bad = torch.tensor([float(device_status(clear=False)[0] != 0)], device="cuda")
            dist.all_reduce(bad)
            assert float(bad) == 0, f"rank {rank}: device status {device_status()}"
            assert float((replayed[:, 11:15] == want[:, 11:15]).float().mean()) >= 0.9
            got = replayed
        # prompt-pass logits: the same numbers up to the all-reduce's summation order
        a, b = record_tp["logits"][0].float(), record["logits"][0].float()
        ok = bool(((a - b).abs() <= 2e-2 * b.abs().max()).all())
        first = slice(11, 15)
        ok = ok and got.shape == want.shape and float((got[:, first] == want[:, first]).float().mean()) >= 0.9
        # all ranks hold the same tokens
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got.contiguous())
        ok = ok and all(torch.equal(gathered[0], t) for t in gathered)
        model._decode_state = None            # captured graphs hold collective kernels: release them before the group goes
        torch.cuda.synchronize()
        ret[rank] = ok
    except BaseException:                                        # noqa: BLE001
        _leave(rank, ret, False)
    _leave(rank, ret, True)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("use_peer", [False, True])
def test_two_gpu_vocab_parallel_model(use_peer):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_model_worker, args=(world, port, ret, use_peer), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
