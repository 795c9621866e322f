"""One engine life cycle on a GPU in a fresh process:

    python tests/engine_check_gpu.py [tp_world_size]

launch_engine starts one worker per GPU (default one, on cuda:0) that builds a small OPT-shaped PipelineModel (seeded);
generation requests (input_ids, attention_mask, max_tokens, top_k=1) travel through the RPC
pipes as the reference's do (energonai/engine.py:79-103, worker.py:74-83); the tokens that come
back must equal those of the same model called directly in this process.  Exit code 0 on success."""
import socket

import torch

from energonai_b200 import launch_engine

KW = dict(vocab_size=1000, max_seq_len=128, hidden_size=256, num_heads=4, depth=2, mlp_ratio=4.0,
          activation=torch.nn.functional.relu, dtype=torch.float16, fused_qkv=False, model_name="opt")


def tiny_opt(**kwargs):
    from energonai_b200.model import PipelineModel
    torch.manual_seed(11)
    return PipelineModel(**kwargs).eval()


def tiny_opt_sharded(**kwargs):
    """The same seeded model cut for this rank of the worker's tensor-parallel group: every rank
    builds the whole (tiny) model under a single-rank context and keeps its own shard."""
    from energonai_b200 import tp
    from energonai_b200.model import PipelineModel
    from energonai_b200.sharding import shard_model_state
    ctx = tp.get_tp()
    tp.set_tp(None)
    full = tiny_opt(**kwargs)
    tp.set_tp(ctx)
    model = PipelineModel(**kwargs).eval()
    model.load_state_dict(shard_model_state(full.state_dict(), ctx.rank, ctx.world_size))
    return model


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def requests():
    g = torch.Generator().manual_seed(5)
    out = {}
    for uid, (batch, length, new) in enumerate(((2, 9, 12), (4, 17, 8), (1, 5, 20))):
        ids = torch.randint(3, 1000, (batch, length), generator=g)
        mask = torch.ones_like(ids)
        mask[0, :2] = 0
        out[uid] = dict(input_ids=ids, attention_mask=mask, max_tokens=length + new, top_k=1)
    return out


def main(tp_world_size=1):
    reqs = requests()
    engine = launch_engine(tp_world_size, 1, "127.0.0.1", free_port(), free_port(),
                           tiny_opt if tp_world_size == 1 else tiny_opt_sharded, **KW)
    try:
        for uid, r in reqs.items():
            engine.submit(uid, r)
        got = {uid: engine.get(uid) for uid in reqs}
    finally:
        engine.shutdown()
    from energonai_b200 import tp
    tp.init_tp(1)
    model = tiny_opt(**KW).cuda()
    for uid, r in reqs.items():
        with torch.inference_mode():
            want = model(**{k: (v.cuda() if torch.is_tensor(v) else v) for k, v in r.items()}).cpu()
        assert got[uid].shape == want.shape
        if tp_world_size == 1:
            assert torch.equal(got[uid], want), (uid, got[uid], want)
        else:
            # a sharded sum adds in another order: near-ties between two logits may resolve
            # differently, after which a sequence continues on its own; the first tokens must agree
            n = r["input_ids"].shape[1]
            agree = float((got[uid][:, n:n + 4] == want[:, n:n + 4]).float().mean())
            assert agree >= 0.9, (uid, agree)
    print(f"engine gpu ok {tp_world_size}", flush=True)


if __name__ == "__main__":
    import sys
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 1)
