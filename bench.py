"""Benchmark of the compiled training step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config bert_tiny] [--impl ours|reference]

One step is one pass of the training step (forward, loss, backward, AdamW) over one synthetic
MLM batch of 32 sequences per GPU. Prints ONE JSON line (rank 0). `value` is batches of 32
sequences trained per second over the whole job with the batch resident in HBM; `e2e` is the same
through the host loop of the C ABI with a new host batch every step (host-to-device copy of the
batch, tokens and scalars, device-to-host read of every loss, inside the timed region).
`roofline` describes the kernel with the largest share of a profiled step; `cpu_baseline` is the
CPU oracle (a port of the reference's single-threaded interpreter) timed on this host.
`--impl reference` times that CPU port alone with every host thread.
"""
import argparse
import datetime
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from modelspec_b200 import models, synthetic  # noqa: E402

METRIC = "train_steps_per_sec"
UNIT = "steps/s (batches of 32 sequences, whole job)"



_LINE_OUT = None  # the descriptor standard output had when the process started (set in main)


def emit_line(record):
    """The one JSON line of a run, on the process's original standard output."""
    data = (json.dumps(record) + "\n").encode()
    if _LINE_OUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_LINE_OUT, data)


def workload(name):
    cfg = models.CONFIGS[name]
    if cfg["kind"] != "bert":
        raise SystemExit("bench.py measures the BERT-shaped configurations")
    return cfg


def ncu_traffic(config, kernel, flop, nbytes):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch from the ncu captures
    summarised under profiles/ (profiles/dram_traffic.json, keyed by workload, plan kernel, and
    the launch's algorithmic FLOP and bytes as the plan reports them); None when no capture of
    that launch is on file."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    entry = json.load(open(path)).get("%s:%s:%d:%d" % (config, kernel, flop, nbytes))
    return entry["dram_bytes"] if entry else None


# The most blocks of --steps steps one invocation times (a short step gets more than --blocks).
kMostBlocks = 40

L2_NOTE = "no explicit flush: every step streams over 1 GB of intermediates through the 126 MB L2"


def config_of(args, cfg, world, masked):
    return {"workload": args.config, "global_batch": cfg["batch"] * world, "seq_len": cfg["seq"], "vocab": cfg["vocab"],
            "masked_rows": masked, "parallelism": "dp%d" % world, "l2": L2_NOTE}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,timestamp")

    def __init__(self, gpu_index):
        # Started before the warm-up (nvidia-smi takes a few hundred milliseconds to deliver its
        # first sample); only the samples between begin() and stop() are kept.
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.begun = time.time()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def begin(self):
        self.begun = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        ended = time.time()
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [l.strip().split(", ") for l in open(self.file.name) if l.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                taken = datetime.datetime.strptime(r[9].strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if taken < self.begun or taken > ended:
                    continue
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_steps(source, masked, vocab, seq, batch, steps, threads, warmup=0):
    """Times `steps` steps of the CPU oracle; returns seconds per step (median)."""
    import oracle_lib
    oracle_lib.lib().orc_set_threads(threads)
    t = oracle_lib.Trainer(source, masked)
    times = []
    for k in range(warmup + steps):
        for name, value in synthetic.mlm_batch(k, vocab=vocab, seq=seq, batch=batch).items():
            t.set_input(name, value)
        t0 = time.perf_counter()
        t.step(k, warmup + steps)
        if k >= warmup:
            times.append(time.perf_counter() - t0)
    oracle_lib.lib().orc_set_threads(os.cpu_count() or 1)
    return float(np.median(times)), times


def reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # The asked steps, bounded so that the run ends within a few minutes (about 2 s a step on 16
    # threads for BERT-tiny).
    steps = max(1, min(args.steps, 40))
    warm = max(0, min(args.warmup, 5))
    source = cfg["source"](steps=steps + warm, warmup_steps=1)
    masked = models.default_masked_rows(cfg["rows"])
    sec, times = cpu_steps(source, masked, cfg["vocab"], cfg["seq"], cfg["batch"], steps, threads, warm)
    value = 1.0 / sec
    sample = ("%d steps (%d warm-up) of one GPU's share of the workload, 32 sequences a step, on the CPU port of the "
              "reference interpreter with %d threads (the interpreter itself is single-threaded)" % (steps, warm, threads))
    emit_line({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": sec * 1e3, "median_ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(args, cfg, args.gpus, masked),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def dp_parity(M, dist, rank, world, local):
    """Outside any timed region: the hidden-32 BERT twin trained for 12 steps sharded over the job's
    ranks through the same library calls as the benchmark (bucketed gradient exchange, global loss
    denominators, dropout indexed in the whole batch), against the CPU oracle's run of the whole
    batch on rank 0. Returns the record rank 0 prints."""
    steps, batch, seq, vocab, capacity = 12, 4, 16, 300, 32
    kw = dict(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=vocab, seq=seq, lr=3e-3, warmup_steps=2, steps=steps)
    rows = batch * seq
    device = M.Device(local)
    run = M.Training(device, models.bert(batch=batch, **kw), capacity)
    ids = [M.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    run.comm_init(rank, world, ids[0], rows)
    feed = lambda k: synthetic.mlm_batch(k, vocab=vocab, seq=seq, batch=batch * world)
    shard = lambda full: {name: value[rank * rows:(rank + 1) * rows] for name, value in full.items()}
    losses = []
    for k in range(steps):
        for name, value in shard(feed(k)).items():
            run.set_input(name, value)
        run.step(k, steps)
        losses.append(float(run.loss()))
    for name, value in shard(feed(steps)).items():
        run.set_input(name, value)
    losses.append(float(run.final_loss()))
    params = [run.step_plan.param_download(i) for i in range(len(run.step_plan.params()))]
    exchange = "peer memory" if M.lib().msx_comm_uses_peer_memory(run.step_plan.h) else "nccl"
    run.destroy()
    device.close()
    record = None
    if rank == 0:
        import oracle_lib
        cpu = oracle_lib.Trainer(models.bert(batch=batch * world, **kw), capacity * world)
        cpu_losses = []
        for k in range(steps):
            for name, value in feed(k).items():
                cpu.set_input(name, value)
            cpu_losses.append(float(cpu.step(k, steps)))
        for name, value in feed(steps).items():
            cpu.set_input(name, value)
        cpu_losses.append(float(cpu.final_loss()))
        # The run tolerance |g - c| <= 1e-4 + 1e-3 |c| on every loss and parameter element (key
        # biases, whose exact gradient is 0, get the reference's steps * lr * 1e-3 on top);
        # `worst_rel` is the largest |g - c| / (that bound), so at most 1 passes.
        worst = 0.0
        g, c = np.array(losses, dtype=np.float64), np.array(cpu_losses, dtype=np.float64)
        worst = max(worst, float(np.max(np.abs(g - c) / (1e-4 + 1e-3 * np.abs(c)))))
        for i, path in enumerate(cpu.param_paths()):
            atol = 1e-4 + steps * 3e-3 * 1e-3 if path.endswith("_bk") else 1e-4
            c = cpu.read("param", i).astype(np.float64)
            worst = max(worst, float(np.max(np.abs(params[i].astype(np.float64) - c) / (atol + 1e-3 * np.abs(c)))))
        record = {"ok": bool(np.isfinite(worst) and worst <= 1.0), "world": world, "worst_rel": worst, "exchange": exchange,
                  "steps": steps, "what": "hidden-32 BERT twin, %d sequences of %d tokens a rank, losses and every parameter "
                                          "against the CPU oracle's whole-batch run" % (batch, seq)}
    return record


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--config", default="bert_tiny")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-steps", type=int, default=2, help="steps of the single-threaded CPU baseline (rank 0, N=1)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--blocks", type=int, default=None,
                    help="how many times the block of --steps steps is timed (default: 7, more for a step so short that "
                         "7 blocks would last under 0.6 s, fewer for one so long that they would last over 20 s)")
    ap.add_argument("--flags", type=int, default=0, help="plan flags (modelspec_b200.PLAN_*)")
    args = ap.parse_args()
    # Standard output carries the one JSON line and nothing else: what libraries print there (NCCL
    # announces its version on stdout) goes to standard error from here on.
    global _LINE_OUT
    sys.stdout.flush()
    _LINE_OUT = os.dup(1)
    os.dup2(2, 1)
    cfg = workload(args.config)
    if args.impl == "reference":
        reference_arm(args, cfg)
        return

    import modelspec_b200 as M

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE is %d" % (args.gpus, world))
    dist = None
    parity = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        parity = dp_parity(M, dist, rank, world, local)

    W, K = max(args.warmup, 3), args.steps
    blocks_asked = max(1, args.blocks if args.blocks is not None else 7)
    total = W + K * (max(blocks_asked, kMostBlocks) + 1)
    end = total + 8
    source = cfg["source"](steps=end, warmup_steps=max(1, total // 10))
    masked = models.default_masked_rows(cfg["rows"])
    device = M.Device(local)
    run = M.Training(device, source, masked, args.flags)
    plan = run.step_plan
    if world > 1:
        # torch.distributed carries the communicator id and the barriers; the gradient
        # all-reduces are the library's own.
        ids = [M.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        run.comm_init(rank, world, ids[0], cfg["rows"])
    stats = plan.stats()
    batch_of = lambda k: synthetic.mlm_batch(k, vocab=cfg["vocab"], seq=cfg["seq"], batch=cfg["batch"],
                                             row_offset=rank * cfg["rows"])

    def barrier():
        plan.sync()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident leg: the batch, tokens and scalars stay staged; no host copy ---------
    # The block of K steps is timed `blocks` times, each between a barrier and a synchronize on
    # both sides, by CUDA events on the plan's stream: one pair around the whole block (the
    # reference's training clock) and one pair around every step (for the median step time).
    for name, value in batch_of(0).items():
        run.set_input(name, value)
    sampler = ClockSampler(local)
    t0 = time.perf_counter()
    for k in range(W):
        run.step(k, end)
    barrier()
    warm_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / W)  # every rank times the same number of blocks
    # A long step (the BERT-base-shaped configuration) gets fewer blocks: about 20 s in all.
    blocks = int(max(1, min(blocks_asked, 20000.0 / max(warm_ms * K, 1e-3))))
    # A short step gets more blocks, so that the timed region lasts long enough (0.6 s) for the
    # clock sampler to see it several times.
    if args.blocks is None:
        last_ms = max_over_ranks(plan.step_ms(plan.steps_submitted() - 1))  # the warm-up's average holds the first step's set-up
        blocks = int(max(blocks, min(kMostBlocks, math.ceil(600.0 / max(last_ms * K, 1e-3)))))
    lag = 4
    sampler.begin()
    block_ms, step_ms = [], []
    for _ in range(blocks):
        barrier()
        plan.elapsed_ms()
        first = plan.steps_submitted()
        for k in range(K):
            plan.run()   # same staged inputs: nothing is uploaded
            if k >= lag:
                step_ms.append(plan.step_ms(first + k - lag))
        for k in range(max(0, K - lag), K):
            step_ms.append(plan.step_ms(first + k))
        ms, counted = plan.elapsed_ms()
        barrier()
        assert counted == K
        block_ms.append(max_over_ranks(ms) / K)
    resident_ms = float(np.median(block_ms))
    median_ms = max_over_ranks(float(np.median(step_ms)))

    # ---- end-to-end leg: a new pinned host batch every step, every loss read back -----------
    batches = [batch_of(W + k) for k in range(K)]
    h2d = stats["upload_bytes_per_step"]
    base = W + K * blocks
    barrier()
    t0 = time.perf_counter()
    plan.elapsed_ms()
    losses = []
    for k in range(K):
        for name, value in batches[k].items():
            run.set_input(name, value)
        run.step(base + k, end)
        if k >= lag:
            losses.append(run.loss_of(base + k - lag))
    for k in range(max(0, K - lag), K):
        losses.append(run.loss_of(base + k))
    e2e_device_ms, _ = plan.elapsed_ms()
    barrier()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(e2e_device_ms, e2e_wall_ms)) / K
    clocks = sampler.stop()   # sampled through both timed legs
    assert all(np.isfinite(l) for l in losses), "a loss of the timed run is not finite"

    exposed_comm_ms = None
    if world > 1:
        barrier()
        exposed_comm_ms = max_over_ranks(float(np.median([plan.comm_exposed_ms() for _ in range(5)])))

    # ---- one profiled step: which launch dominates, its roofline, and the step's ---------------
    # Every launch is issued 10 times back to back between two CUDA events on the plan's stream
    # and its time divided by 10 (a few-microsecond launch is otherwise timed at the host's
    # launch rate). The roofline object describes the single heaviest launch of the step;
    # roofline.step compares the whole step with the time its launches would take at the measured
    # peaks: max(flop / tensor peak, bytes / HBM rate) for the contractions, bytes / HBM rate for
    # the rest, FLOP and bytes by the reference's counting rule.
    barrier()
    prof = plan.profile_step(10)
    by_kernel = {}
    for kernel, ms, nbytes, flop in prof:
        e = by_kernel.setdefault(kernel, {"launches": 0, "ms": 0.0, "bytes": 0, "flop": 0})
        e["launches"] += 1; e["ms"] += ms; e["bytes"] += nbytes; e["flop"] += flop
    profiled_ms = sum(e["ms"] for e in by_kernel.values())
    top_kernel, top_ms, top_bytes, top_flop = max(prof, key=lambda launch: launch[1])
    pk = peaks()
    contractions = ("matmul", "matmul_jobs", "attention_forward", "attention_backward")
    half = bool(args.flags & M.PLAN_BF16) if hasattr(M, "PLAN_BF16") else False
    t_roof_ms = 0.0
    for kernel, ms, nbytes, flop in prof:
        t_bytes = nbytes / (pk["hbm_gbs"] * 1e9) * 1e3
        t_flop = flop / (pk["bf16_tflops"] * 1e12) * 1e3 if kernel in contractions else 0.0
        t_roof_ms += max(t_bytes, t_flop)
    traffic = ncu_traffic(args.config, top_kernel, top_flop, top_bytes)
    if top_flop and top_kernel in contractions:
        achieved = top_flop / (top_ms * 1e-3) / 1e12
        roofline = {"kernel": top_kernel, "bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / pk["bf16_tflops"], "traffic": traffic,
                    "hbm_view": {"achieved_gbs": top_bytes / (top_ms * 1e-3) / 1e9, "peak_gbs": pk["hbm_gbs"],
                                 "frac": top_bytes / (top_ms * 1e-3) / 1e9 / pk["hbm_gbs"]}}
        if not half:
            # f32 products on the tf32 tensor cores take three partial products each (hi/lo split
            # of both operands; lo x lo is left out), and dense tf32 runs at half the bf16 rate:
            # the ceiling of this kernel class is 1/6 of the measured bf16 peak.
            roofline["frac_of_split_tf32_ceiling"] = achieved / (pk["bf16_tflops"] / 6)
    else:
        achieved = top_bytes / (top_ms * 1e-3) / 1e9
        roofline = {"kernel": top_kernel, "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "traffic": traffic}
    roofline.update({"peak_source": pk["source"], "launch_ms": top_ms, "share_of_step": top_ms / profiled_ms,
                     "algorithmic_bytes": top_bytes, "algorithmic_flop": top_flop,
                     "kernel_class": {"launches_per_step": by_kernel[top_kernel]["launches"], "ms_per_step": by_kernel[top_kernel]["ms"],
                                      "share_of_step": by_kernel[top_kernel]["ms"] / profiled_ms},
                     "step": {"t_roof_ms": t_roof_ms, "ms_per_step": resident_ms, "frac": t_roof_ms / resident_ms}})
    shares = {kname: round(v["ms"] / profiled_ms, 4) for kname, v in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"])}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        src = cfg["source"](steps=args.cpu_steps, warmup_steps=1)
        sec, _ = cpu_steps(src, masked, cfg["vocab"], cfg["seq"], cfg["batch"], args.cpu_steps, 1)
        cpu_baseline = {"value": 1.0 / sec, "unit": UNIT, "cores": 1, "kind": "port", "ms_per_step": sec * 1e3,
                        "sample": "%d full steps of the same workload, single thread as the reference interpreter runs" % args.cpu_steps}

    if rank == 0:
        line = {
            "metric": METRIC, "value": world * 1e3 / resident_ms, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": resident_ms, "median_ms_per_step": median_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if half else "f32", "data": "synthetic",
            "tokens_per_sec": world * cfg["rows"] * 1e3 / resident_ms,
            "config": config_of(args, cfg, world, masked),
            "blocks": {"count": blocks, "steps_each": K, "ms_per_step_median": resident_ms, "ms_per_step_min": min(block_ms),
                       "ms_per_step_max": max(block_ms), "timed_steps": len(step_ms)},
            "clocks": clocks,
            "e2e": {"value": world * 1e3 / e2e_ms, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 8, "losses_read": len(losses)},
            "gpu_launches": stats["launches_per_step"] * K,
            "launches_per_step": stats["launches_per_step"],
            "roofline": roofline, "kernel_shares": shares, "profiled_step_ms": profiled_ms,
            "algorithmic_bytes_per_step": stats["algorithmic_bytes_per_step"],
            "matmul_flop_per_step": stats["matmul_flop_per_step"],
            "cpu_baseline": cpu_baseline,
        }
        if world > 1:
            line["data_parallel"] = {
                "gradient_buckets": int(M.lib().msx_comm_bucket_count(plan.h)),
                "gradient_exchange": "peer memory" if M.lib().msx_comm_uses_peer_memory(plan.h) else "nccl",
                "exposed_comm_ms": exposed_comm_ms}
            line["dp_parity"] = parity
        emit_line(line)
    run.destroy()
    device.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
