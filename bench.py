"""Benchmark of the tensor-parallel transformer layer path: OPT-13B-shaped fp16 generation.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One "step" = one pass of the hot path over one batch: the prompt pass (batch 16, 512
left-padded positions) plus 128 greedy generation steps through all 40 layers, with the
model sharded over N GPUs (tensor parallel, heads and FFN columns).  Rank 0 prints one JSON
line.  Inputs are synthetic and weights random-init (seeded); the weights alone (26 GB) are
larger than L2, so consecutive timed steps cannot reuse cached data.

`--impl reference` times the reference's own algorithm for this path (its PyTorch layer
forward, restated in oracle/layers.py) on the host CPU cores, on a bounded sample of the
same workload, and prints the same line with "impl": "reference".
"""
import argparse
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
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
def build_model(cfg, dtype):
    import torch
    from energonai_b200.model import create_pipeline_model
    torch.manual_seed(1234)          # same seed on every rank: replicated parameters agree
    with torch.device("cuda"):
        model = create_pipeline_model(depth=cfg["depth"], vocab_size=cfg["vocab"], hidden_size=cfg["hidden"],
                                      max_seq_len=cfg["max_pos"], num_heads=cfg["heads"],
                                      mlp_ratio=cfg["ffn"] / cfg["hidden"], activation=torch.nn.functional.relu,
                                      is_decoder=True, fused_qkv=False, dtype=dtype)
    with torch.no_grad():
        model.embed.word_embeddings.weight.normal_(0, 0.02)
        model.embed.position_embeddings.weight.normal_(0, 0.02)
    return model.eval()


def probe_decode_gemms(model, cfg):
    """Average device time per launch of the generation-step GEMM (the dominant kernel).

    All four GEMMs of every layer are launched back to back, with each layer's own weights (so
    every launch streams weights that are not in L2), captured in one CUDA graph and replayed;
    CUDA events on the launching stream bracket each replay.  Returns (algorithmic bytes, ms,
    launches) per replay."""
    import torch
    from energonai_b200.gemm import gemm
    B, h = cfg["batch"], cfg["hidden"]
    dt = model.norm.module.weight.dtype
    x = torch.randn(B, h, device="cuda", dtype=dt)
    jobs = []
    for blk in model.blocks:
        w_qkv, _ = blk.attn._packed()
        jobs += [(x, w_qkv), (torch.randn(B, blk.attn.dense.weight.shape[1], device="cuda", dtype=dt), blk.attn.dense.weight),
                 (x, blk.mlp.dense_1.weight),
                 (torch.randn(B, blk.mlp.dense_2.weight.shape[1], device="cuda", dtype=dt), blk.mlp.dense_2.weight)]

    def run():
        for a, w in jobs:
            gemm(a, w, static_weight=True)

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
    nbytes = sum((w.shape[0] * w.shape[1] + a.shape[0] * a.shape[1] + a.shape[0] * w.shape[0]) * 2 for a, w in jobs)
    return nbytes, e0.elapsed_time(e1) / reps, len(jobs)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from energonai_b200 import _lib, tp
    from oracle import inputs   # seeded prompt generator only (no oracle compute on this path)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        ctx = tp.init_tp(world)
        if os.environ.get("EB_PEER", "1") != "0":
            # generation steps: all-reduce fused into the row-parallel GEMM epilogue (NVLink peer stores)
            try:
                ctx.enable_peer_exchange(CFG["batch"], CFG["hidden"])
            except Exception as e:          # no peer mapping on this box: NCCL carries every all-reduce
                ctx.peer = None
                if rank == 0:
                    print(f"peer exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
    cfg = dict(CFG)
    if args.layers:
        cfg["depth"] = args.layers
    if args.new_tokens:
        cfg["new_tokens"] = args.new_tokens
    model = build_model(cfg, torch.float16)
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
    t_wall = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        out_h = one(False)
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t_wall) * 1e3 * 0)   # device time; the .cpu() read is synchronous

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = t.tolist()

    # per-phase figures from the step events of the timed region (rank 0's own clock)
    prefill_ms, step_ms = [], []
    for rec in recs:
        ev = rec["step_events"]
        prefill_ms.append(ev[0].elapsed_time(ev[1]))
        step_ms += [a.elapsed_time(b) for a, b in zip(ev[1:-1], ev[2:])]
    peak, peak_kind = measured_peaks()
    roof = None
    if rank == 0 or world > 1:
        gemm_bytes, gemm_ms, gemm_n = probe_decode_gemms(model, cfg)
        achieved = gemm_bytes / (gemm_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                # dram__bytes_read+write per launch from the ncu capture summarised in
                # profiles/gemm_decode_opt13b_m16.md (same four shapes, full-size launches)
                "traffic": 162.0e6 if (world == 1 and not args.layers) else None, "kernel": "gemm_kernel<__half, 16, true> (generation-step GEMM, M = batch 16)",
                "peak_kind": f"of {peak_kind}", "launches_timed": gemm_n,
                "algorithmic_bytes_per_launch": gemm_bytes / max(1, gemm_n), "us_per_launch": gemm_ms * 1e3 / max(1, gemm_n)}
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
    ms_per_step = elapsed_ms / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "config": workload_config(world),
            "prefill_tokens_per_s": cfg["batch"] * cfg["prompt"] / (statistics.mean(prefill_ms) * 1e-3),
            "decode_tokens_per_s": cfg["batch"] / (statistics.mean(step_ms) * 1e-3) if step_ms else None,
            "decode_step_ms_p50": statistics.median(step_ms) if step_ms else None,
            "prefill_ms": statistics.mean(prefill_ms),
            "e2e": {"value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": ids_h.numel() * ids_h.element_size() + mask_h.numel() * mask_h.element_size(),
                    "d2h_bytes_per_step": out_h.numel() * out_h.element_size()},
            "gpu_launches": launches, "clocks": clocks, "roofline": roof}
    if world == 1 and not args.no_cpu:
        v, sample, cores, _ = cpu_sample(CFG)
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    if args.layers or args.new_tokens:
        line["config"]["reduced"] = f"depth {cfg['depth']}, new_tokens {cfg['new_tokens']} (debug run, not the named config)"
    print(json.dumps(line), flush=True)
    finish()


def main():
    if os.environ.get("EB_BENCH_WATCHDOG"):       # debugging aid: dump all Python stacks if the run stalls
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ["EB_BENCH_WATCHDOG"]), repeat=False, exit=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (marks the line as reduced)")
    ap.add_argument("--new-tokens", type=int, default=0, help="debug: fewer generation steps (marks the line as reduced)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
