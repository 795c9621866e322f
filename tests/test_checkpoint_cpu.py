"""Checkpoint conversion and loading (energonai/utils/checkpointing*.py) on CPU: the renamed
state dicts equal the ones the reference's own converters produce (committed fixture, and live
where a checkout of the reference is present); a whole-model checkpoint loads into one rank and
into two gloo ranks, whose shards together are the checkpoint again."""
import json
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import checkpoint_cases as cc  # noqa: E402

from energonai_b200 import utils as U  # noqa: E402

with open(os.path.join(HERE, "golden", "checkpoint_names.json")) as f:
    GOLDEN = json.load(f)


@pytest.mark.parametrize("case", sorted(cc.CASES))
def test_converters_equal_the_reference_fixture(case):
    build, conv = cc.CASES[case]
    got = cc.summarise(getattr(U, conv)(build()))
    want = GOLDEN[case]
    assert [g[0] for g in got] == [w[0] for w in want]              # names, in order
    assert [g[1] for g in got] == [w[1] for w in want]              # shapes
    for g, w in zip(got, want):
        assert g[2] == pytest.approx(w[2], rel=1e-9, abs=1e-6), g[0]  # values (transposes, chunks)


@pytest.mark.parametrize("case", sorted(cc.CASES))
def test_converters_equal_the_reference_live(case):
    from oracle import ref_loader
    if ref_loader.reference_root() is None or ref_loader.load_reference_model_package() is None:
        pytest.skip("reference checkout not present")
    import importlib
    build, conv = cc.CASES[case]
    mod = "energonai.utils.checkpointing_hf_gpt2" if conv == "processing_HF_GPT" else "energonai.utils.checkpointing_opt"
    ref = getattr(importlib.import_module(mod), conv)(build())
    mine = getattr(U, conv)(build())
    if conv == "processing_HF_GPT":
        assert mine["epoch"] == ref["epoch"] == 0
        ref, mine = ref["model"], mine["model"]
    assert list(ref) == list(mine)
    for k in ref:
        assert torch.equal(ref[k], mine[k]), k


def test_opt_keys_under_another_root_fail_like_the_reference():
    # processing_OPT only knows the `decoder.` root; with `model.decoder.` the embedding is not
    # found when the head is cloned from it (KeyError in the reference as well)
    with pytest.raises(KeyError):
        U.processing_OPT(cc.opt_hf(root="model.decoder."))


def test_remove_prefix():
    out = U.remove_prefix({"model.a.b": 1, "c": 2}, "model")
    assert list(out.items()) == [("a.b", 1), ("c", 2)]


DIMS = dict(vocab_size=cc.V, hidden_size=cc.H * 16, depth=cc.L, num_heads=2, max_seq_len=cc.P, dtype=torch.float32)


def _opt_checkpoint(h, f, with_head=False):
    """Hugging Face style OPT checkpoint of the DIMS model."""
    gen = torch.Generator().manual_seed(5)
    t = lambda *s: torch.randn(*s, generator=gen) * 0.1  # noqa: E731
    d = {"decoder.embed_tokens.weight": t(cc.V, h), "decoder.embed_positions.weight": t(cc.P, h)}
    for i in range(cc.L):
        p = f"decoder.layers.{i}."
        for n in ("self_attn_layer_norm", "final_layer_norm"):
            d[p + n + ".weight"], d[p + n + ".bias"] = t(h), t(h)
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            d[p + f"self_attn.{n}.weight"], d[p + f"self_attn.{n}.bias"] = t(h, h), t(h)
        d[p + "fc1.weight"], d[p + "fc1.bias"], d[p + "fc2.weight"], d[p + "fc2.bias"] = t(f, h), t(f), t(h, f), t(h)
    d["decoder.final_layer_norm.weight"], d["decoder.final_layer_norm.bias"] = t(h), t(h)
    return d


def _build(**kw):
    from energonai_b200.model.model_factory import create_pipeline_model
    model_kwargs = dict(DIMS, activation=torch.nn.functional.relu, fused_qkv=False, is_decoder=True)
    model_kwargs.update(kw)
    return create_pipeline_model(**model_kwargs)


@pytest.mark.skipif(torch.cuda.is_available(), reason="builds the model on the CPU")
@pytest.mark.parametrize("as_dir", [False, True])
def test_load_checkpoint_single_rank(tmp_path, as_dir, monkeypatch):
    h = DIMS["hidden_size"]
    ckpt = _opt_checkpoint(h, 4 * h)
    if as_dir:
        path = tmp_path / "parts"
        path.mkdir()
        keys = list(ckpt)
        for n, part in enumerate((keys[:7], keys[7:20], keys[20:])):
            torch.save({k: ckpt[k] for k in part}, path / f"part{n}.pt")
        monkeypatch.setenv("LOAD_N_PROC", "2")
    else:
        path = tmp_path / "opt.pt"
        torch.save(ckpt, path)
    model = _build(checkpoint=str(path), model_name="opt")
    want = U.processing_OPT(dict(ckpt))
    got = model.state_dict()
    assert set(got) == set(want)
    for k in want:
        assert torch.equal(got[k], want[k]), k
    # the head starts as a copy of the embedding, not as the same storage
    assert got["head.dense.weight"].data_ptr() != got["embed.word_embeddings.weight"].data_ptr()
    with pytest.raises(FileNotFoundError):
        _build(checkpoint=str(tmp_path / "missing.pt"), model_name="opt")
    with pytest.raises(RuntimeError):       # strict: an entry the model does not have
        torch.save(dict(ckpt, **{"decoder.layers.0.extra.weight": torch.zeros(1)}), tmp_path / "bad.pt")
        _build(checkpoint=str(tmp_path / "bad.pt"), model_name="opt")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, path, vocab_parallel, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from energonai_b200 import tp as tpmod
        tpmod.init_tp(world)
        model = _build(checkpoint=path, model_name="opt", vocab_parallel=vocab_parallel)
        ret[rank] = {k: v.clone() for k, v in model.state_dict().items()}
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.is_available(), reason="builds the model on the CPU")
@pytest.mark.parametrize("vocab_parallel", [False, True])
def test_load_checkpoint_two_ranks_reassemble_the_checkpoint(tmp_path, vocab_parallel):
    h = DIMS["hidden_size"]
    ckpt = _opt_checkpoint(h, 4 * h)
    path = str(tmp_path / "opt.pt")
    torch.save(ckpt, path)
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_tp_worker, args=(world, port, path, vocab_parallel, ret), nprocs=world, join=True)
    full = U.processing_OPT(dict(ckpt))
    shards = [ret[r] for r in range(world)]
    assert set(shards[0]) == set(full)
    for k, v in full.items():
        a, b = shards[0][k], shards[1][k]
        if a.shape == v.shape:                                   # replicated
            assert torch.equal(a, v) and torch.equal(b, v), k
        elif a.shape[0] * 2 == v.shape[0]:                       # column-parallel / vocabulary rows
            assert torch.equal(torch.cat([a, b], 0), v), k
        else:                                                    # row-parallel weight
            assert a.dim() == 2 and a.shape[1] * 2 == v.shape[1], k
            assert torch.equal(torch.cat([a, b], 1), v), k
    cut = {k for k in full if shards[0][k].shape != full[k].shape}
    assert any("attn.query_.weight" in k for k in cut) and any("mlp.dense_2.weight" in k for k in cut)
    assert ("embed.word_embeddings.weight" in cut) == vocab_parallel
    assert ("head.dense.weight" in cut) == vocab_parallel


@pytest.mark.skipif(torch.cuda.is_available(), reason="builds the model on the CPU")
def test_load_175b_part_and_gpt2(tmp_path):
    from energonai_b200.model.model_factory import create_pipeline_model
    # one rank's part of the resharded 175B format: fused key | value | query rows, norm names
    # without the LayerNorm1D wrapper level
    h, f = DIMS["hidden_size"], 4 * DIMS["hidden_size"]
    gen = torch.Generator().manual_seed(9)
    t = lambda *s: torch.randn(*s, generator=gen)  # noqa: E731
    part = {"decoder.embed_tokens.weight": t(cc.V, h), "decoder.embed_positions.weight": t(cc.P, h),
            "decoder.layer_norm.weight": t(h), "decoder.layer_norm.bias": t(h)}
    for i in range(cc.L):
        p = f"decoder.layers.{i}."
        for n, shape in (("self_attn_layer_norm", (h,)), ("final_layer_norm", (h,)), ("self_attn.qkv_proj", (3 * h, h)),
                         ("self_attn.out_proj", (h, h)), ("fc1", (f, h)), ("fc2", (h, f))):
            part[p + n + ".weight"], part[p + n + ".bias"] = t(*shape), t(shape[0])
    d = tmp_path / "175b"
    d.mkdir()
    torch.save(part, d / "reshard-model_part-0.pt")
    model = create_pipeline_model(**dict(DIMS, activation=torch.nn.functional.relu, fused_qkv=True,
                                         checkpoint=str(d), model_name="opt-175b"))
    got = model.state_dict()
    assert torch.equal(got["blocks.1.attn.query_key_value.weight"], part["decoder.layers.1.self_attn.qkv_proj.weight"])
    assert torch.equal(got["blocks.0.norm2.module.bias"], part["decoder.layers.0.final_layer_norm.bias"])
    assert torch.equal(got["norm.module.weight"], part["decoder.layer_norm.weight"])
    assert torch.equal(got["head.dense.weight"], part["decoder.embed_tokens.weight"])

    # Hugging Face GPT-2: Conv1D layouts transposed, c_attn cut into query_ / key_ / value_
    g = {"wte.weight": t(cc.V, h), "wpe.weight": t(cc.P, h), "ln_f.weight": t(h), "ln_f.bias": t(h)}
    for i in range(cc.L):
        p = f"h.{i}."
        for n, shape in (("ln_1", (h,)), ("ln_2", (h,)), ("attn.c_attn", (h, 3 * h)), ("attn.c_proj", (h, h)),
                         ("mlp.c_fc", (h, f)), ("mlp.c_proj", (f, h))):
            g[p + n + ".weight"], g[p + n + ".bias"] = t(*shape), t(shape[-1])
        g[p + "attn.bias"] = torch.ones(1, 1, cc.P, cc.P)
    torch.save(g, tmp_path / "gpt2.pt")
    model = create_pipeline_model(**dict(DIMS, fused_qkv=False, checkpoint=str(tmp_path / "gpt2.pt"),
                                         model_name="hf_gpt2"))
    got = model.state_dict()
    assert torch.equal(got["blocks.0.attn.key_.weight"], g["h.0.attn.c_attn.weight"].t()[h:2 * h])
    assert torch.equal(got["blocks.1.attn.value_.bias"], g["h.1.attn.c_attn.bias"][2 * h:])
    assert torch.equal(got["blocks.1.mlp.dense_2.weight"], g["h.1.mlp.c_proj.weight"].t())
    assert torch.equal(got["blocks.0.norm1.module.weight"], g["h.0.ln_1.weight"])
    assert torch.equal(got["norm.module.bias"], g["ln_f.bias"])
