"""Benchmark of the sparse MLA attention operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one call of the operator on one batch of seeded synthetic input. The default
workload is the prefill configuration the reference's headline numbers are quoted on: B=1,
8192 queries at the end of a 32768-token context, H=64, D=512, TopK=512 of a 2x-compressed
cache plus a 128-token window, BF16. With N > 1 (one process per GPU under torchrun) every
rank runs its own replica of the workload with its own seed: no data-path collective, weak
scaling; `value` is the work of all ranks over the slowest rank's time.

Timing mirrors the reference's protocol (its README.md:56-58): CUDA events bracket each
attention launch on the launching stream, an eviction pass writing four times the L2 size
runs before every timed launch, input preparation is outside the timed region.

`--impl reference` times the reference's CPU numerical reference (the oracle port) on the host
cores for the same workload, on a bounded sample of query tokens.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "sparse_mla_effective_tflops_qk_pv_fma2"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# dram__bytes_read.sum + dram__bytes_write.sum of the attention kernel per query token, from the
# ncu captures summarised under profiles/: prefill Q8K/ctx32K (1090.1 MB for 8192 tokens) and
# decode B16 x 6 queries at ctx 128K (58.97 MB for 96 tokens). Other sizes of the same regime are
# scaled by token count, since traffic is Q + O + gathered rows per token.
MEASURED_TRAFFIC_PER_TOKEN = {"prefill": 1087.22e6 / 8192, "decode": 59.10e6 / 96}
L2_BYTES = 126 * 1024 * 1024


def parse():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200", choices=("b200", "reference"))
    parser.add_argument("--workload", default="prefill_q8k_ctx32k")
    parser.add_argument("--cpu-sample-seconds", type=float, default=12.0)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    return parser.parse_args()


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", 0.0))}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples of one GPU while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.process = index, [], None
        self.window = [None, None]  # host times bracketing the region whose samples count

    def mark_begin(self):
        self.window[0] = time.time()

    def mark_end(self):
        self.window[1] = time.time()

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._drain, daemon=True).start()
        except OSError:
            self.process = None
        return self

    def _drain(self):
        for line in self.process.stdout:
            self.lines.append((time.time(), line.strip()))

    def __exit__(self, *error):
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self):
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        begin, end = self.window
        for stamp, line in self.lines:
            if begin is not None and (stamp < begin or (end is not None and stamp > end + 0.05)):
                continue
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 7:
                continue
            try:
                clocks.append(float(fields[0]))
                maxima.append(float(fields[1]))
            except ValueError:
                continue
            for name, state in zip(names, fields[3:7]):
                if state.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima),
                "reasons": sorted(reasons), "samples": len(clocks)}


def policy_of(config):
    from oracle import sparse_mla_oracle as O

    return O.make_policy(config["batches"], config["batches"] * config["queries"], max_seq=config["max_seq"])


def cpu_reference_rate(meta_and_rows, policy, budget_seconds, threads):
    """Time the oracle's FP32 torch-CPU form on as many sampled tokens as fit the budget.

    `meta_and_rows(tokens)` returns (q, sinks, rows per token). Returns the record and the
    seconds per live row, from which a whole-call time is extrapolated.
    """
    import numpy as np
    import torch
    from oracle import sparse_mla_oracle as O

    torch.set_num_threads(threads)
    tokens_total = policy["T"]
    rng = np.random.default_rng(17)
    probe = sorted(rng.choice(tokens_total, size=min(32, tokens_total), replace=False).tolist())
    q, sinks, rows = meta_and_rows(probe)
    small = dict(policy, T=len(probe))
    O.reference_fp32(q, sinks, lambda i: rows[i], small, chunk=32)  # warm the BLAS threads
    start = time.perf_counter()
    O.reference_fp32(q, sinks, lambda i: rows[i], small, chunk=32)
    probe_seconds = time.perf_counter() - start
    per_token = probe_seconds / len(probe)
    count = int(max(len(probe), min(tokens_total, budget_seconds / max(per_token, 1e-6))))
    count = min(count, 4096)
    sample = sorted(rng.choice(tokens_total, size=count, replace=False).tolist())
    q, sinks, rows = meta_and_rows(sample)
    small = dict(policy, T=count)
    start = time.perf_counter()
    O.reference_fp32(q, sinks, lambda i: rows[i], small, chunk=128)
    seconds = time.perf_counter() - start
    live = sum(len(r) for r in rows)
    flops = 4 * policy["H"] * policy["D"] * live
    return {
        "value": flops / seconds / 1e12,
        "unit": UNIT,
        "cores": threads,
        "kind": "port",
        "sample": (f"{count} of {tokens_total} query tokens drawn uniformly (seed 17), {live} live rows, "
                   f"{seconds:.2f} s; FP32 torch-CPU bmm/softmax/bmm in chunks of 128 queries "
                   "(the reference's numerical reference, restated for the CPU)"),
        "seconds": seconds,
        "seconds_per_call_extrapolated": None,
    }, seconds / max(live, 1)


def host_rows_provider(config, seed, sigma=1.0):
    """Rows for sampled tokens without a GPU: metadata from the workload generator; cache rows
    are gathered by physical row id (modulo the pool size) from a seeded N(0, sigma) pool, which
    gives a CPU timing the right shapes, gather pattern and value distribution."""
    import numpy as np
    from ascendflow_b200 import workloads as W
    from oracle import sparse_mla_oracle as O

    meta, live = W.host_metadata(config["batches"], config["queries"], config["context"], config["max_seq"], 2, seed)
    policy = policy_of(config)

    pool_rows = 1 << 15
    rng = np.random.default_rng(seed + 1)
    pool = O.round_b16(rng.normal(0, sigma, (pool_rows, 512)).astype(np.float32), "bf16")
    q_pool = O.round_b16(rng.normal(0, sigma, (256, 64, 512)).astype(np.float32), "bf16")

    def provide(tokens):
        resolved = O.resolve_rows(meta, policy, tokens)
        q = q_pool[np.asarray(tokens) % len(q_pool)]
        rows = [pool[ids[ids >= 0] % pool_rows] for ids in resolved]
        return q, np.linspace(-2, 2, 64, dtype=np.float32), rows

    return provide, policy, live


def run_reference(args, config):
    """The reference arm: its CPU numerical reference on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    provide, policy, live = host_rows_provider(config, 4102026)
    # steps/warmup bound the work: each step is one bounded sample.
    budget = max(2.0, min(args.cpu_sample_seconds, 120.0 / max(1, args.steps + args.warmup)))
    records = []
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_reference_rate(provide, policy, min(budget, 2.0), threads)
    for _ in range(max(1, min(args.steps, 3))):
        record, per_row = cpu_reference_rate(provide, policy, budget, threads)
        records.append((record, per_row))
    record, per_row = max(records, key=lambda item: item[0]["value"])
    seconds_per_call = per_row * live
    record["seconds_per_call_extrapolated"] = seconds_per_call
    value = record["value"]
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds_per_call * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": args.workload, **config,
                                        "note": "CPU time per call extrapolated from the sampled tokens"},
        "cpu_baseline": record,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_b200(args, config):
    import numpy as np
    import torch
    import torch.distributed as dist

    from ascendflow_b200 import ops, workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU fallback"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    warmup = max(args.warmup, 3)

    tensors, meta, work = W.device_case(**config, seed=4102026 + rank, device=device)
    call = ops.kernel("sparse_mla").bind(*tensors.values())
    flush = torch.empty(4 * L2_BYTES, dtype=torch.uint8, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        flush.zero_()
        call()
    barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local) as clocks:
        time.sleep(0.3)  # let the sampler come up before the region starts
        barrier()
        clocks.mark_begin()
        for step in range(args.steps):
            flush.zero_()
            starts[step].record()
            binding = call()
            ends[step].record()
        barrier()
        timed_seconds = time.time() - clocks.window[0]
        # nvidia-smi samples every 100 ms: when the timed region is shorter than a second, the same
        # launches keep running (untimed) so that the clock record covers the same load.
        hold_steps = 0
        while time.time() - clocks.window[0] < 1.2:
            flush.zero_()
            call()
            hold_steps += 1
            if hold_steps % 8 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        clocks.mark_end()
    durations = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    status = binding.status()
    assert status[0] == 0, f"kernel status block reports {status}"
    mean_ms = sum(durations) / len(durations)
    slowest = torch.tensor([mean_ms], dtype=torch.float64, device=device)
    total_flops = torch.tensor([float(work["flops"])], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_flops, op=dist.ReduceOp.SUM)
    ms_per_step = float(slowest.item())
    value = float(total_flops.item()) / (ms_per_step * 1e-3) / 1e12

    # End to end through the public op with host buffers: every step copies the step's inputs
    # (queries, indices, tables, lengths) from pinned memory and reads the whole output back.
    # The paged KV caches are the operator's resident state and stay on the device.
    e2e = None
    if not args.no_e2e:
        moving = ("q", "cmp_sparse_indices", "ori_block_table", "cmp_block_table", "cu_seqlens_q",
                  "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length", "sinks")
        pinned = {name: tensors[name].cpu().pin_memory() for name in moving}
        h2d = sum(t.numel() * t.element_size() for t in pinned.values())
        d2h = tensors["attention_out"].numel() * tensors["attention_out"].element_size()
        # Two sets of step tensors so that the copy-in of step i + 1, the kernel of step i and the
        # copy-out of step i - 1 overlap on three streams, as a serving loop would run them.
        sets = []
        for _ in range(2):
            own = dict(tensors)
            for name in moving + ("attention_out",):
                own[name] = torch.empty_like(tensors[name])
            sets.append((own, torch.empty(tensors["attention_out"].shape,
                                          dtype=tensors["attention_out"].dtype).pin_memory()))
        copy_in, compute, copy_out = (torch.cuda.Stream(device=device) for _ in range(3))
        consumed = [None, None]   # kernel of the step that last used the set has finished
        drained = [None, None]    # its output has reached the host

        def e2e_step(index):
            own, host_out = sets[index % 2]
            with torch.cuda.stream(copy_in):
                if consumed[index % 2] is not None:
                    copy_in.wait_event(consumed[index % 2])
                for name in moving:
                    own[name].copy_(pinned[name], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(arrived)
                if drained[index % 2] is not None:
                    compute.wait_event(drained[index % 2])
                ops.sparse_mla(*own.values())
                consumed[index % 2] = torch.cuda.Event()
                consumed[index % 2].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(consumed[index % 2])
                host_out.copy_(own["attention_out"], non_blocking=True)
                drained[index % 2] = torch.cuda.Event()
                drained[index % 2].record(copy_out)

        steps = max(4, min(args.steps, 12))
        for index in range(2):
            e2e_step(index)
        barrier()
        wall = time.perf_counter()
        for index in range(steps):
            e2e_step(index)
        barrier()
        e2e_ms = torch.tensor([(time.perf_counter() - wall) * 1e3 / steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        e2e = {"value": float(total_flops.item()) / (float(e2e_ms.item()) * 1e-3) / 1e12, "unit": UNIT,
               "ms_per_step": float(e2e_ms.item()), "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "note": "public op (torch custom-op path) with host buffers: every step copies queries, indices, "
                       "tables and lengths from pinned memory and reads the whole output back; copy-in, kernel "
                       "and copy-out of neighbouring steps overlap on three streams; KV caches are the "
                       "operator's resident state; timed by host clock between device synchronisations"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, source = peaks()
    own_ms = mean_ms
    decode = config["queries"] <= 16
    if decode:
        achieved = work["unique_bytes"] / (own_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peak["hbm_gbs"],
                    "traffic": MEASURED_TRAFFIC_PER_TOKEN["decode"] * work["tokens"],
                    "traffic_source": "ncu capture of decode_b16_q6_ctx128k scaled by tokens"}
    else:
        achieved = work["flops"] / (own_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peak["bf16_tflops"],
                    "traffic": MEASURED_TRAFFIC_PER_TOKEN["prefill"] * work["tokens"],
                    "traffic_source": "ncu capture of prefill_q8k_ctx32k scaled by tokens"}
    roofline["peak_source"] = f"{source} (burst figure: each launch is timed alone between L2 evictions)"
    roofline["kernel"] = "sparse_mla attention kernel, one launch per step"
    roofline["algorithmic"] = {"flops_per_launch": work["flops"], "unique_bytes_per_launch": work["unique_bytes"],
                               "logical_bytes_per_launch": work["logical_bytes"]}
    roofline["logical_gather_gbs"] = work["logical_bytes"] / (own_ms * 1e-3) / 1e9

    record = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, **config, "heads": 64, "features": 512, "topk": 512,
                   "window": 128, "ratio": 2, "values": "N(0,1)", "seed": 4102026,
                   "replicas": world, "l2": "evicted before every timed launch (504 MiB written)",
                   "timing": "CUDA events around each launch; mean of steps; max over ranks",
                   "ms_per_step_min": min(durations), "ms_per_step_median": statistics.median(durations)},
        "roofline": roofline,
        "clocks": dict(clocks.summary(), region=f"timed region ({timed_seconds:.2f} s) plus {hold_steps} identical "
                                                "untimed launches so that the 100 ms sampler sees the load"),
        "gpu_launches": args.steps,
    }
    if e2e is not None:
        record["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        policy = policy_of(config)
        def provide(tokens):
            import numpy as np
            from oracle import sparse_mla_oracle as O

            resolved = O.resolve_rows(meta, policy, tokens)
            ori = tensors["ori_kv"].view(-1, 512)
            cmp = tensors["cmp_kv"].view(-1, 512)
            rows = []
            for ids in resolved:
                head, tail = ids[:128], ids[128:]
                head, tail = head[head >= 0], tail[tail >= 0]
                rows.append(np.concatenate([
                    ori[torch.as_tensor(head, device=device)].float().cpu().numpy(),
                    cmp[torch.as_tensor(tail, device=device)].float().cpu().numpy()]))
            q = tensors["q"][torch.as_tensor(np.asarray(tokens), device=device)].float().cpu().numpy()
            return q, tensors["sinks"].float().cpu().numpy(), rows

        baseline, per_row = cpu_reference_rate(provide, policy, args.cpu_sample_seconds, os.cpu_count() or 1)
        baseline["seconds_per_call_extrapolated"] = per_row * work["live_rows"]
        record["cpu_baseline"] = baseline
    print(json.dumps(record))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    from ascendflow_b200 import workloads as W

    if args.workload not in W.CONFIGS:
        raise SystemExit(f"unknown workload {args.workload}; choose from {sorted(W.CONFIGS)}")
    config = dict(W.CONFIGS[args.workload])
    if args.impl == "reference":
        run_reference(args, config)
    else:
        run_b200(args, config)


if __name__ == "__main__":
    main()
