"""Benchmark of the tensor-parallel transformer layer path: OPT-13B-shaped fp16 generation.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One "step" = one pass of the hot path over one batch: the prompt pass (batch 16, 512
left-padded positions) plus 128 greedy generation steps through all 40 layers, with the
model sharded over N GPUs (tensor parallel, heads and FFN columns).  Rank 0 prints one JSON
line.  Inputs are synthetic and weights random-init (seeded); the weights alone (26 GB) are
larger than L2, so consecutive timed steps cannot reuse cached data.

Besides timing, the run verifies what it timed (outside the timed region): all ranks must
hold identical tokens, no bounded device-side wait may have run out, and a two-layer model of
the same layer shape, sharded the same way, must reproduce the CPU oracle's greedy tokens and
final hidden states ("check" in the line).

`--impl reference` times the reference's own algorithm for this path (its PyTorch layer
forward, restated in oracle/layers.py) on the host CPU cores, on a bounded sample of the
same workload, and prints the same line with "impl": "reference".
"""
import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(name="OPT-13B", hidden=5120, heads=40, ffn=20480, depth=40, vocab=50272, max_pos=2050,
           batch=16, prompt=512, new_tokens=128, len_lo=256)
METRIC = "OPT-13B fp16 tokens/s (prefill+decode)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm": float(d["hbm_gbs"]), "tensor": float(d["bf16_tflops"]),
                "tensor_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
    return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        if not sm:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference algorithm (oracle port) on a bounded sample
# ------------------------------------------------------------------------------------------------
def cpu_sample(cfg, decode_steps=3):
    """One of the `depth` layers, fp32, on all host cores: the prompt pass, then `decode_steps`
    generation steps (each re-runs attention over the whole sequence, as the reference does).
    Returns (estimated tokens/s of the whole job, description, cores)."""
    import torch
    from oracle import inputs, layers
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(0)
    bp = inputs.block_params(gen, cfg["hidden"], cfg["ffn"])
    B, S = cfg["batch"], cfg["prompt"]
    x = torch.randn(B, S + decode_steps, cfg["hidden"], generator=gen)
    lens = torch.randint(cfg["len_lo"], S + 1, (B,), generator=gen)
    mask = (torch.arange(S)[None, :] >= (S - lens)[:, None]).float()
    blk = layers.OracleBlock(bp, cfg["heads"], "relu")
    with torch.inference_mode():
        t0 = time.perf_counter()
        blk(x[:, :S], (1.0 - mask.view(B, 1, 1, S)) * -10000.0, True)
        t_prefill = time.perf_counter() - t0
        t_dec = []
        for i in range(1, decode_steps + 1):
            m = torch.cat([mask, torch.ones(B, i)], 1)
            t0 = time.perf_counter()
            blk(x[:, :S + i], (1.0 - m.view(B, 1, 1, S + i)) * -10000.0, False)
            t_dec.append(time.perf_counter() - t0)
    t_job = cfg["depth"] * (t_prefill + cfg["new_tokens"] * statistics.median(t_dec))
    tokens = B * (S + cfg["new_tokens"])
    sample = (f"1 of {cfg['depth']} layers in fp32: prompt pass (batch {B} x {S}) {t_prefill:.2f} s + {decode_steps} "
              f"generation steps (median {statistics.median(t_dec):.3f} s); job time extrapolated as "
              f"{cfg['depth']} x (prompt + {cfg['new_tokens']} x step)")
    return tokens / t_job, sample, cores, t_job


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_sample(CFG, decode_steps=1)
    vals, jobs = [], []
    for _ in range(args.steps):
        v, sample, cores, t_job = cpu_sample(CFG)
        vals.append(v)
        jobs.append(t_job)
    value = statistics.mean(vals)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.mean(jobs) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    c = CFG
    return {"workload": f"{c['name']}-shaped decoder, random init: {c['depth']} layers, hidden {c['hidden']}, "
                        f"{c['heads']} heads, FFN {c['ffn']} ReLU; batch {c['batch']}, prompts left-padded to "
                        f"{c['prompt']} (true lengths uniform in [{c['len_lo']},{c['prompt']}]), prompt pass + "
                        f"{c['new_tokens']} greedy steps with KV cache",
            "global_batch": c["batch"], "seq_len": c["prompt"], "new_tokens": c["new_tokens"],
            "parallelism": f"tp{n_gpus}", "l2": "inputs larger than L2 (26 GB of weights stream every step)"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def build_model(cfg, dtype, world):
    import torch
    from energonai_b200.model import create_pipeline_model
    torch.manual_seed(1234)          # same seed on every rank: replicated parameters agree
    with torch.device("cuda"):
        # on a tensor-parallel group the vocabulary is split too (the reference does that for its
        # largest factory, model_factory.py:352): every rank streams 1/N of the LM head per step
        model = create_pipeline_model(depth=cfg["depth"], vocab_size=cfg["vocab"], hidden_size=cfg["hidden"],
                                      max_seq_len=cfg["max_pos"], num_heads=cfg["heads"],
                                      mlp_ratio=cfg["ffn"] / cfg["hidden"], activation=torch.nn.functional.relu,
                                      is_decoder=True, fused_qkv=False, dtype=dtype, vocab_parallel=world > 1)
    with torch.no_grad():
        model.embed.word_embeddings.weight.normal_(0, 0.02)
        model.embed.position_embeddings.weight.normal_(0, 0.02)
    return model.eval()


def step_bytes(cfg, world, kv_len):
    """Algorithmic bytes one generation step moves on ONE rank: this rank's weight shards, its
    slice of the cached keys and values, the LM head it streams."""
    h, f, e = cfg["hidden"], cfg["ffn"], 2
    weights = cfg["depth"] * (4 * h * h + 2 * h * f) * e / world
    kv = cfg["depth"] * 2 * cfg["batch"] * kv_len * h * e / world
    head = cfg["vocab"] * h * e / world
    return weights + kv + head


def probe_decode_kernels(model, cfg, st, world):
    """Average device time per launch of the dominant generation-step kernel, launched with the
    step's real arguments (folded LayerNorms, bias, residual, cache-row mapping, the exchange of
    a tensor-parallel group), back to back, each layer on its own weights (nothing is
    L2-resident), captured in one CUDA graph and replayed between CUDA events.

    Single rank: the four GEMMs of every layer (eb_gemm_ln for QKV / FC1, eb_gemm with bias and
    residual for out-proj / FC2).  Tensor-parallel group: the chained launches of the step (one
    per layer: out-proj, exchange, FC1, FC2, exchange, QKV).  Returns a dict."""
    import torch
    B, h = cfg["batch"], cfg["hidden"]
    dt = model.norm.module.weight.dtype
    e = 2
    if st.get("chains"):
        chains = st["chains"]

        def run():
            for ch in chains:
                ch.run()
        n_launch = len(chains)
        nbytes = cfg["depth"] * (4 * h * h + 2 * h * cfg["ffn"]) * e / world + cfg["vocab"] * h * e / world
        name = "chain_kernel<__half, 16> (one launch per layer: out-proj, exchange + LayerNorm, FC1, FC2, exchange + LayerNorm, QKV)"
    else:
        from energonai_b200.gemm import gemm
        x = torch.randn(B, 1, h, device="cuda", dtype=dt)
        kv_state = st["kv_state"]
        jobs = []
        nbytes = 0
        for blk in model.blocks:
            at, mlp = blk.attn, blk.mlp
            w, b = at._packed()
            w_f, colsum, bias32, eps = at._fold.get(w, b, blk.norm1, at._param_versions())
            buf = at.past_cache.buf
            ctx = torch.randn(B, 1, at.local_hidden, device="cuda", dtype=dt)
            jobs.append(lambda w_f=w_f, colsum=colsum, bias32=bias32, eps=eps, buf=buf: gemm(
                x[:, 0], w_f, static_weight=True, out=buf, out_rows_per_batch=1, out_batch_stride=buf.stride(0),
                out_ld=buf.stride(1), out_row_offset_device=kv_state[0:1], out_row_limit=buf.shape[1],
                ln_fold=(colsum, bias32, eps)))
            jobs.append(lambda at=at, ctx=ctx: at.dense(ctx, residual=x))
            jobs.append(lambda mlp=mlp, blk=blk: mlp.dense_1(x, act=mlp.act_code, fold_norm=blk.norm2))
            inter = torch.randn(B, 1, mlp.dense_1.out_per_rank, device="cuda", dtype=dt)
            jobs.append(lambda mlp=mlp, inter=inter: mlp.dense_2(inter, residual=x))
            for wt, k_in in ((w, h), (at.dense.weight, at.local_hidden), (mlp.dense_1.weight, h),
                             (mlp.dense_2.weight, mlp.dense_1.out_per_rank)):
                nbytes += (wt.numel() + B * k_in + B * wt.shape[0]) * e

        def run():
            for j in jobs:
                j()
        n_launch = len(jobs)
        name = "gemm_kernel<__half, 16, true> (generation-step GEMM, M = batch 16; QKV / FC1 with the LayerNorm folded in)"
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    g.replay()
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"kernel": name, "bytes": nbytes, "ms": ms, "launches": n_launch}


def exposed_exchange(model, cfg, ids_d, mask_d, tgt, prefill_ms, step_ms):
    """How much of the prompt pass and of the generation step is spent waiting for the other
    ranks: the same shards, shapes and launches are timed once more with the exchange reduced to
    this rank alone (a context of one rank that exchanges with itself; NCCL all-reduces skipped),
    so the numbers it produces are meaningless but nothing waits for a peer.
    exposed fraction = (time with the exchange - time without) / time with."""
    import torch
    from energonai_b200 import tp
    from energonai_b200.comm import PeerExchange
    ctx = tp.get_tp()
    real_peer, real_all_reduce, real_gather = ctx.peer, ctx.all_reduce, ctx.all_gather_last_dim
    from energonai_b200._lib import lib
    line_b, bulk_b = (real_peer.line_bytes, real_peer.bulk_bytes) if real_peer is not None else (1 << 20, 0)
    area = torch.zeros(lib().eb_comm_area_bytes(line_b, bulk_b), dtype=torch.uint8, device="cuda")
    solo = PeerExchange.from_pointers(0, 1, area, [area.data_ptr()], line_bytes=line_b)
    solo.max_rows, solo.max_cols = cfg["batch"], cfg["hidden"]
    saved_state = model._decode_state
    try:
        if real_peer is not None:
            ctx.peer = solo
        ctx.all_reduce = lambda t: t
        ctx.all_gather_last_dim = lambda t: torch.cat([t] * ctx.world_size, dim=-1)
        model._decode_state = None
        rec = {"allow_graph": True}
        model(input_ids=ids_d, attention_mask=mask_d, max_tokens=tgt, top_k=1, record=rec)
        model(input_ids=ids_d, attention_mask=mask_d, max_tokens=tgt, top_k=1, record=(rec := {"allow_graph": True}))
        torch.cuda.synchronize()
        ev = rec["step_events"]
        solo_prefill = ev[0].elapsed_time(ev[1])
        solo_steps = [a.elapsed_time(b) for a, b in zip(ev[1:-1], ev[2:])]
    finally:
        ctx.peer, ctx.all_reduce, ctx.all_gather_last_dim = real_peer, real_all_reduce, real_gather
        model._decode_state = saved_state
        from energonai_b200.gemm import device_status
        device_status(clear=True)
        solo.destroy()
    solo_step = statistics.median(solo_steps) if solo_steps else None
    out = {"prefill_ms_without_exchange": solo_prefill, "decode_step_ms_without_exchange": solo_step,
           "exposed_allreduce_frac_prefill": max(0.0, (prefill_ms - solo_prefill) / prefill_ms)}
    if solo_step and step_ms:
        out["exposed_allreduce_frac_decode"] = max(0.0, (step_ms - solo_step) / step_ms)
    return out


def verify(world, rank, out_tokens):
    """Checks on what was timed, outside the timed region.  Returns a dict for the line."""
    import torch
    import torch.distributed as dist
    from energonai_b200 import tp
    from energonai_b200.gemm import device_status
    from energonai_b200.sharding import shard_model_state
    from oracle import inputs, layers      # the checker (never on the timed path)
    res = {}
    problems = []
    tok = out_tokens.contiguous()
    res["tokens_sha"] = hashlib.sha256(tok.cpu().numpy().tobytes()).hexdigest()[:16]
    if world > 1:
        gathered = [torch.empty_like(tok) for _ in range(world)]
        dist.all_gather(gathered, tok)
        if not all(torch.equal(gathered[0], t) for t in gathered):
            problems.append("ranks hold different tokens")
    st = device_status(clear=True)
    peer = tp.get_tp().peer
    cst = peer.status() if peer is not None else (0, 0, 0, 0)
    bad = torch.tensor([1.0 if (st[0] != 0 or cst[0] != 0) else 0.0], device="cuda")
    if world > 1:
        dist.all_reduce(bad)
    if float(bad) > 0:
        problems.append(f"a device-side wait ran out or a limit was hit on some rank (this rank: {st}, {cst})")

    # two layers of the benchmark's layer shape, sharded like the benchmark, against the CPU oracle
    c = dict(vocab=2048, max_pos=128, hidden=CFG["hidden"], heads=CFG["heads"], ffn=CFG["ffn"], depth=2, B=CFG["batch"], S=32, new=5)
    from energonai_b200.model import PipelineModel
    p = inputs.model_params(3, c["vocab"], c["max_pos"], c["hidden"], c["ffn"], c["depth"], rich=True)
    ids, mask, _ = inputs.left_padded_prompts(3, c["B"], c["S"], c["S"] // 2, c["S"], c["vocab"])
    tgt = c["S"] + c["new"]
    full = {k: v.half() for k, v in layers.model_to_reference_state(p, c["depth"], False).items()}
    with torch.device("cuda"):
        small = PipelineModel(vocab_size=c["vocab"], max_seq_len=c["max_pos"], hidden_size=c["hidden"], num_heads=c["heads"],
                              depth=c["depth"], mlp_ratio=c["ffn"] / c["hidden"], activation=torch.nn.functional.relu,
                              dtype=torch.float16, fused_qkv=False, vocab_parallel=world > 1).eval()
    small.load_state_dict(shard_model_state(full, rank, world, vocab_parallel=world > 1), strict=True)
    del full
    got = small(input_ids=ids.cuda(), attention_mask=mask.cuda(), max_tokens=tgt, top_k=1)      # replayed steps
    res["check_step_launch"] = (small._decode_state or {}).get("chain_mode") or "one kernel per operation"
    if rank == 0:
        rec = {}
        with torch.inference_mode():
            want = layers.OracleModel(p, c["depth"], c["heads"], "relu").generate(ids, mask, tgt, rec)
        logits = torch.stack(rec["logits"], 0)
        top2 = logits.topk(2, -1).values
        margin = (top2[..., 0] - top2[..., 1])              # [new, B]
        got_c, ok_seqs = got.cpu(), 0
        for b in range(c["B"]):
            diff = (got_c[b, c["S"]:] != want[b, c["S"]:]).nonzero()
            if diff.numel() == 0:
                ok_seqs += 1
            elif float(margin[int(diff[0]), b]) >= 2e-2:
                problems.append(f"sequence {b} leaves the oracle's greedy tokens at step {int(diff[0])} "
                                f"(margin {float(margin[int(diff[0]), b]):.3g})")
        res["check_sequences_identical"] = f"{ok_seqs}/{c['B']}"
    st = device_status(clear=True)
    if st[0] != 0:
        problems.append(f"device status after the check run: {st}")
    del small
    torch.cuda.empty_cache()
    flag = torch.tensor([float(len(problems))], device="cuda")
    if world > 1:
        dist.all_reduce(flag)
    res["check"] = "ok" if float(flag) == 0 else "FAILED: " + "; ".join(problems or ["see another rank"])
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from energonai_b200 import tp
    from oracle import inputs   # seeded prompt generator only (no oracle compute on the timed path)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    cfg = dict(CFG)
    if args.layers:
        cfg["depth"] = args.layers
    if args.new_tokens:
        cfg["new_tokens"] = args.new_tokens
    exchange_kind = "none (one rank)"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        ctx = tp.init_tp(world)
        exchange_kind = "NCCL all-reduce"
        if os.environ.get("EB_PEER", "1") != "0":
            # generation steps: the all-reduces run inside the library's own kernels over NVLink peer memory
            try:
                bulk = cfg["batch"] * cfg["prompt"] if os.environ.get("EB_PEER_PROMPT", "1") != "0" else 0
                ctx.enable_peer_exchange(128, cfg["hidden"], bulk_rows=bulk)
                exchange_kind = ("prompt pass: " + ("reduce-scatter in the GEMM epilogue + reduce/broadcast kernel, NVLink peer stores"
                                                    if bulk else "NCCL all-reduce") +
                                 "; generation steps: inside the chained kernel, NVLink peer stores")
            except Exception as e:          # no peer mapping on this box: NCCL carries every all-reduce
                ctx.peer = None
                if rank == 0:
                    print(f"peer exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
    model = build_model(cfg, torch.float16, world)
    ids_h, mask_h, _ = inputs.left_padded_prompts(0, cfg["batch"], cfg["prompt"], cfg["len_lo"], cfg["prompt"], cfg["vocab"])
    ids_h, mask_h = ids_h.pin_memory(), mask_h.pin_memory()
    ids_d, mask_d = ids_h.cuda(), mask_h.cuda()
    tgt = cfg["prompt"] + cfg["new_tokens"]
    tokens_per_step = cfg["batch"] * tgt

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one(resident, rec=None):
        if resident:
            return model(input_ids=ids_d, attention_mask=mask_d, max_tokens=tgt, top_k=1, record=rec)
        out = model(input_ids=ids_h.cuda(non_blocking=True), attention_mask=mask_h.cuda(non_blocking=True),
                    max_tokens=tgt, top_k=1)
        return out.cpu()

    for _ in range(args.warmup):
        one(True)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    recs, launches = [], 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        rec = {"allow_graph": True}
        out = one(True, rec)
        recs.append(rec)
        launches += model.launches_last_call
    ev1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = ev0.elapsed_time(ev1)
    assert out.shape == (cfg["batch"], tgt), out.shape

    # the same metric end to end: host (pinned) inputs in, host tokens out, copies inside the timed region
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out_h = one(False)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)          # device time; the .cpu() read of the tokens is synchronous

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = t.tolist()

    # per-phase figures from the step events of the timed region (this rank's own clock)
    prefill_ms, step_ms = [], []
    for rec in recs:
        ev = rec["step_events"]
        prefill_ms.append(ev[0].elapsed_time(ev[1]))
        step_ms += [a.elapsed_time(b) for a, b in zip(ev[1:-1], ev[2:])]
    prefill_mean = statistics.mean(prefill_ms)
    step_p50 = statistics.median(step_ms) if step_ms else None
    peaks = measured_peaks()

    # ---- explanations, outside the timed region ----
    probe = probe_decode_kernels(model, cfg, model._decode_state, world)
    exposed = exposed_exchange(model, cfg, ids_d, mask_d, tgt, prefill_mean, step_p50) if world > 1 else None
    checks = verify(world, rank, out) if not args.no_check else {"check": "skipped"}

    def finish():
        # Captured graphs hold NCCL kernels; tearing the process group down under them can
        # block, so release the graphs, rendezvous once more and leave without the teardown.
        if world > 1:
            model._decode_state = None
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        finish()
        return
    achieved = probe["bytes"] / (probe["ms"] * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "decode_gemm_dram_bytes_per_launch.txt")
    if world == 1 and not args.layers and os.path.exists(tpath):
        with open(tpath) as f:            # dram__bytes_read.sum + dram__bytes_write.sum per launch, from an ncu capture
            traffic = float(f.read().split()[0])
    roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
            "traffic": traffic, "kernel": probe["kernel"], "peak_kind": f"of {peaks['kind']}",
            "launches_timed": probe["launches"], "algorithmic_bytes_per_launch": probe["bytes"] / max(1, probe["launches"]),
            "us_per_launch": probe["ms"] * 1e3 / max(1, probe["launches"])}
    if step_p50:
        kv_mid = cfg["prompt"] + cfg["new_tokens"] // 2
        whole = step_bytes(cfg, world, kv_mid) / (step_p50 * 1e-3) / 1e9
        roof["whole_step"] = {"algorithmic_bytes_per_rank": step_bytes(cfg, world, kv_mid), "achieved": whole, "frac": whole / peaks["hbm"],
                              "note": "weights + keys/values + LM head of one rank / decode_step_ms_p50"}
    h, f, T = cfg["hidden"], cfg["ffn"], cfg["batch"] * cfg["prompt"]
    prompt_flops = cfg["depth"] * (2 * T * h * (4 * h + 2 * f) + 4 * cfg["batch"] * cfg["prompt"] ** 2 * h / 2) / world
    roof["prompt_pass"] = {"bound": "tensor", "achieved": prompt_flops / (prefill_mean * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "peak": peaks["tensor_sustained"], "frac": prompt_flops / (prefill_mean * 1e-3) / 1e12 / peaks["tensor_sustained"],
                           "note": "GEMM + causal-useful attention flops of one rank / prefill_ms, against the sustained bf16 GEMM peak"}
    ms_per_step = elapsed_ms / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    config = workload_config(world)
    config["exchange"] = exchange_kind
    config["lm_head"] = "vocabulary split over the ranks" if world > 1 else "replicated"
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "config": config,
            "prefill_tokens_per_s": cfg["batch"] * cfg["prompt"] / (prefill_mean * 1e-3),
            "decode_tokens_per_s": cfg["batch"] / (statistics.mean(step_ms) * 1e-3) if step_ms else None,
            "decode_step_ms_p50": step_p50, "prefill_ms": prefill_mean,
            "e2e": {"value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": ids_h.numel() * ids_h.element_size() + mask_h.numel() * mask_h.element_size(),
                    "d2h_bytes_per_step": out_h.numel() * out_h.element_size()},
            "gpu_launches": launches, "clocks": clocks, "roofline": roof}
    line.update(checks)
    if exposed:
        line.update(exposed)
    if world == 1 and not args.no_cpu:
        v, sample, cores, _ = cpu_sample(CFG)
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    if args.layers or args.new_tokens:
        line["config"]["reduced"] = f"depth {cfg['depth']}, new_tokens {cfg['new_tokens']} (debug run, not the named config)"
    print(json.dumps(line), flush=True)
    finish()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (marks the line as reduced)")
    ap.add_argument("--new-tokens", type=int, default=0, help="debug: fewer generation steps (marks the line as reduced)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the verification against the oracle")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
