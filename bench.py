#!/usr/bin/env python
"""Benchmark of the training hot path: samples/s of one full step (forward + backward + gradient
all-reduce + Adam) of the large causal Transformer, on N B200s of one node.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
  python bench.py --impl reference ...                     times the CPU path on the host cores

One JSON line is printed by rank 0.  A "step" is one TrainBatch over the global batch of 256 sequences
(sharded evenly over the ranks: strong scaling).  `value` is measured with inputs resident in HBM and
CUDA events on the library's stream; `e2e` through the host-buffer entry point (H2D of ids and one-hot
targets from pinned memory and the loss read back inside the timed region).  The inputs are synthetic
(seeded token ids, uniform) and the weights random-init of the named architecture.  The activations of
one step (tens of GB) are far larger than the 126 MB L2, so no explicit flush is needed between steps."""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from goneuron_b200 import configs, descriptors as D  # noqa: E402

WORKLOADS = {
    "transformer_large": dict(name="transformer_large", kw={}, global_batch=256),
    "transformer_small": dict(name="transformer_small", kw={}, global_batch=64),
    "mlp": dict(name="mlp", kw={}, global_batch=64),
    "cnn": dict(name="cnn", kw={}, global_batch=128),
    "lstm": dict(name="lstm", kw={}, global_batch=256),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm_gbs=j["hbm_gbs"], bf16_tflops=j["bf16_tflops"], bf16_tflops_sustained=j["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons)}


def cpu_sample_large_transformer(kw_full, threads, seed=7, check_linearity=True):
    """Bounded CPU sample of the large-transformer step: `threads` sequences through the full-width model
    with 0 and with 1 of its 8 identical blocks (embedding + positional table + CLS + vocabulary head in
    both), timed on `threads` worker threads like the reference's worker pool; the per-sequence cost of the
    full model is t0 + n_blocks * (t1 - t0).  With `check_linearity` a third point (2 blocks) is timed as well
    and the residual (t2 - t1) / (t1 - t0) - 1 of the straight line is returned, so the extrapolation is
    checked in the same run."""
    from oracle import binding as oracle
    times = {}
    for nb in ((0, 1, 2) if check_linearity else (0, 1)):
        kw = dict(kw_full); kw["n_blocks"] = nb
        layers, loss_kind = configs.transformer(**kw)
        rng = np.random.Generator(np.random.PCG64(seed))
        params = configs.init_params(layers, rng)
        x, y = configs.make_inputs("transformer_large", layers, threads, rng)
        st = oracle.OracleState(layers, loss_kind, params, lr=1e-4)
        st.train_batch(x, y, W=threads, threads=threads, precision=32)
        times[nb] = st.seconds
    per_block = max(times[1] - times[0], 1e-9)
    per_batch = times[0] + kw_full["n_blocks"] * per_block
    residual = (times[2] - times[1]) / per_block - 1.0 if check_linearity else None
    return threads / per_batch, times, residual


def cpu_baseline(workload, threads, budget_s=30.0, check_linearity=True):
    """samples/s of the CPU restatement of the reference path (kind "port") on `threads` host threads."""
    from oracle import binding as oracle
    oracle.build()
    fn, kw, batch, lr = configs.CONFIGS[workload["name"]]
    kw = dict(kw); kw.update(workload["kw"])
    if workload["name"] == "transformer_large":
        v, times, res = cpu_sample_large_transformer(kw, threads, check_linearity=check_linearity)
        txt = (f"{threads} sequences of 512 tokens through the full-width model with 0 and 1 of 8 blocks (t0={times[0]:.2f}s, t1={times[1]:.2f}s), "
               f"extrapolated to 8 blocks")
        if res is not None:
            txt += f"; linearity checked with a third point, 2 blocks: t2={times[2]:.2f}s, (t2-t1)/(t1-t0)-1 = {res:+.3f}"
        return v, txt
    layers, loss_kind, params, x, y, lr = configs.make_case(workload["name"], **workload["kw"])
    st = oracle.OracleState(layers, loss_kind, params, lr=lr)
    n = x.shape[0]
    st.train_batch(x[:min(n, threads)], y[:min(n, threads)], W=threads, threads=threads, precision=32)
    per = st.seconds / min(n, threads)
    take = int(max(threads, min(n, budget_s / max(per, 1e-9) * threads / 2)))
    take = min(n, take)
    st.train_batch(x[:take], y[:take], W=threads, threads=threads, precision=32)
    return take / st.seconds, f"one step over {take} of {n} samples, {threads} worker threads"


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    # Every step is one bounded sample of the workload.  The whole run is kept within a few minutes: once the
    # time budget is spent the remaining steps are not executed and the line says how many were.
    vals, sample, t_start, budget = [], "", time.perf_counter(), 200.0
    warm = min(args.warmup, 1)
    first_sample = ""
    for i in range(warm + args.steps):
        v, sample = cpu_baseline(workload, threads, budget_s=8.0, check_linearity=(i == 0))     # the straight line is checked once per run
        if i == 0:
            first_sample = sample
        if i >= warm:
            vals.append(v)
        if time.perf_counter() - t_start > budget and vals:
            break
    sample = first_sample + f"; {len(vals)} of {args.steps} timed steps executed within the {budget:.0f} s budget"
    value = len(vals) / sum(1.0 / v for v in vals)
    line = {
        "impl": "reference", "metric": "train samples/s (fwd+bwd+Adam)", "value": value, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * workload["global_batch"] / value, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload["name"], "global_batch": workload["global_batch"], "note": "CPU restatement of the reference's Go CPU path (no Go toolchain on this image); every step is a bounded sample"},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


def measure_tf32_peak(seconds=1.5):
    """Dense TF32 throughput of the box, measured like the driver's bf16 figure: torch.matmul on 8192^3 fp32 operands
    with TF32 allowed, best of 10 (burst) and back to back for `seconds` (sustained).  Outside every timed region."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda"); b = torch.randn(n, n, device="cuda")
        for _ in range(3):
            a @ b
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); a @ b; e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(seconds * 1e3 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            a @ b
        e1.record(); torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        return {"tf32_tflops": flops / (best * 1e-3) / 1e12, "tf32_tflops_sustained": flops * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12,
                "how": f"torch.matmul fp32 {n}^3 with TF32 allowed: best of 10 and {reps} back to back"}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


# DRAM traffic of the contraction kernel from one ncu capture (dram__bytes_read.sum + dram__bytes_write.sum of one
# gemm_tc_persist_kernel<256> launch, M = 16384 tokens, N = K = 1024, on the 32-sequence case; see the summary of that
# capture under profiles/): measured bytes over the launch's algorithmic bytes.  Traffic grows in proportion with the
# operand and output sizes, so a full step's figure is this ratio times the step's algorithmic bytes.
# (Below 1: most of the 67 MB output is still in the 126 MB L2 when the launch ends and is written back later.)
NCU_TRAFFIC_RATIO = {"captured_bytes": 71.455744e6 + 24.339968e6, "algorithmic_bytes": 4.0 * (16384 + 1024) * 1024 + 4.0 * 16384 * 1024}


def run_workload(torch, dist, dev, workload, rank, world, local, steps, warmup, e2e=True, sampler=None):
    """Times one workload on this context: device-resident steps (CUDA events on the library's stream), a profiled pass
    for the contraction roofline, and the same step end to end from pinned host buffers."""
    from goneuron_b200.sequential import Adam, Sequential
    from goneuron_b200.sharding import shard_bounds

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    GB = workload["global_batch"]
    first, last = shard_bounds(GB, rank, world)
    B = last - first
    layers, loss_kind, _, lr = configs.build(workload["name"], **workload["kw"])
    rng = np.random.Generator(np.random.PCG64(configs.SEEDS[workload["name"]]))
    params = configs.init_params(layers, rng)
    xg, yg = configs.make_inputs(workload["name"], layers, GB, rng)
    x, y = xg[first:first + B], yg[first:first + B]
    del xg, yg
    model = Sequential(layers, dev).Compile(Adam(lr), loss_kind)
    model.SetParams(params)
    x_dev, y_dev = dev.alloc(x), dev.alloc(y)

    # ---- device-resident timing (value) -----------------------------------------------------
    for _ in range(warmup):
        model.TrainBatchDevice(x_dev, y_dev, B, GB, first)
    barrier()
    if sampler:
        sampler.start()
    # The large Transformer streams tens of GB per step, far beyond the 126 MB L2.  The other workloads would sit in
    # L2 from one step to the next, so for them every timed step is preceded by an L2 flush (a 256 MB write) and
    # timed on its own.
    flush = workload["name"] != "transformer_large"
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    launches = 0
    if flush:
        ms = 0.0
        for _ in range(steps):
            flush_buf.zero_()
            torch.cuda.synchronize()
            dev.timer_start()
            loss = model.TrainBatchDevice(x_dev, y_dev, B, GB, first)
            ms += dev.timer_stop()
            launches += model.stats().kernel_launches
    else:
        dev.timer_start()
        for _ in range(steps):
            loss = model.TrainBatchDevice(x_dev, y_dev, B, GB, first)
            launches += model.stats().kernel_launches
        ms = dev.timer_stop()
    barrier()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms], device="cuda")
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())

    # ---- contraction roofline: per-launch CUDA events over a profiled pass ------------------
    model.set_profiling(1)
    model.TrainBatchDevice(x_dev, y_dev, B, GB, first)
    gms, gfl, gl, ar_ms, gby, sby = 0.0, 0.0, 0, 0.0, 0.0, 0.0
    for _ in range(2):
        if flush:
            flush_buf.zero_(); torch.cuda.synchronize()
        model.TrainBatchDevice(x_dev, y_dev, B, GB, first)
        st = model.stats()
        gms += st.gemm_ms; gfl += st.gemm_flops; gl += st.gemm_launches; ar_ms += st.allreduce_ms; gby += st.gemm_bytes; sby += st.split_bytes
    model.set_profiling(0)
    prof = dict(gemm_ms=gms / 2, gemm_flops=gfl / 2, gemm_launches=gl // 2, allreduce_ms=ar_ms / 2, gemm_bytes=gby / 2, split_bytes=sby / 2)

    # ---- end to end through the host-buffer entry point ---------------------------------------
    e2e_out = None
    if e2e:
        xp = torch.from_numpy(x).pin_memory().numpy()
        yp = torch.from_numpy(y).pin_memory().numpy()
        model.TrainBatch(xp, yp, GB, first)
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            model.TrainBatch(xp, yp, GB, first)
        torch.cuda.synchronize()
        el = time.perf_counter() - t0
        tt = torch.tensor([el], device="cuda")
        if dist:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_out = {"value": GB * steps / float(tt.item()), "unit": "samples/s",
                   "h2d_bytes_per_step": int(x.nbytes + y.nbytes) * world, "d2h_bytes_per_step": 8 * world}
    barrier()
    model.Close()
    dev.free(x_dev); dev.free(y_dev)
    return dict(GB=GB, B=B, params=int(params.size), ms_total=ms_total, loss=loss, launches=int(launches), clocks=clocks, prof=prof, e2e=e2e_out, flush=flush)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="transformer_large", choices=sorted(WORKLOADS))
    ap.add_argument("--global-batch", type=int, default=0, help="override the global batch (profiling a smaller case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-side-configs", action="store_true", help="skip the short runs of the four smaller benchmark configs")
    args = ap.parse_args()
    workload = dict(WORKLOADS[args.workload])
    if args.global_batch > 0:
        workload["global_batch"] = args.global_batch
    if args.impl == "reference":
        return run_reference(args, workload)

    import torch
    from goneuron_b200.sequential import Device
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt = torch.frombuffer(bytearray(Device.unique_id()), dtype=torch.uint8).cuda()
        dist.broadcast(idt, 0)
        dev = Device(local, rank, world, bytes(idt.cpu().numpy().tobytes()))
    else:
        dev = Device(local)

    r = run_workload(torch, dist, dev, workload, rank, world, local, args.steps, args.warmup, e2e=not args.no_e2e,
                     sampler=ClockSampler(local) if rank == 0 else None)
    GB, ms_total = r["GB"], r["ms_total"]
    value = GB * args.steps / (ms_total / 1e3)
    pk = peaks()
    pf = r["prof"]
    achieved = pf["gemm_flops"] / (pf["gemm_ms"] / 1e3) / 1e12 if pf["gemm_ms"] > 0 else 0.0
    ratio = NCU_TRAFFIC_RATIO["captured_bytes"] / NCU_TRAFFIC_RATIO["algorithmic_bytes"] if NCU_TRAFFIC_RATIO["captured_bytes"] else None
    operand_elems_bytes = pf["split_bytes"] / 2.0           # 4 B per fp32 operand element that went through a split pass
    roofline = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / pk["bf16_tflops_sustained"],
                "traffic": ratio * pf["gemm_bytes"] if ratio else None,
                "traffic_note": "DRAM bytes of the step's contraction launches: ncu-measured bytes / algorithmic bytes of one captured launch (32-sequence case) times the step's algorithmic bytes",
                "algorithmic_bytes_per_step": pf["gemm_bytes"],
                "kernel": "contraction kernel launches of the step (gemm_tc_persist_kernel: three fp16 tcgen05 MMAs per fp32 product on row-scaled split planes; small shapes on the fp32 SIMT kernel), CUDA events around each launch",
                "flops_per_step": pf["gemm_flops"], "launches_per_step": pf["gemm_launches"], "ms_per_step": pf["gemm_ms"], "allreduce_ms_per_step": pf["allreduce_ms"],
                "frac_of_scheme_ceiling": achieved / (pk["bf16_tflops_sustained"] / 3.0),
                "split_passes": {"bytes_per_step": pf["split_bytes"], "fp32_operand_bytes_per_step": operand_elems_bytes,
                                 "operand_traffic_ratio": (pf["split_bytes"] + operand_elems_bytes) / operand_elems_bytes if operand_elems_bytes else None,
                                 "note": "bytes moved by the separate split passes that are left (4 B read + 4 B written per element they handle; weight matrices once per update); operands whose planes are written by their producer -- the LayerNorm kernels, the plane-writing contraction epilogues -- do not appear here"},
                "peak_source": pk["source"] + " cuBLAS bf16 (sustained); an fp32-accurate product here is three fp16 MMAs (fp16 and bf16 run at the same rate), so its arithmetic ceiling is 1/3 of this"}

    side, tf32 = None, None
    if rank == 0 and world == 1:
        tf32 = measure_tf32_peak()
        roofline["tf32_peak_measured"] = tf32
        roofline["frac_of_tf32_sustained_over_3"] = achieved / (tf32["tf32_tflops_sustained"] / 3.0)
    if world == 1 and not args.no_side_configs and args.workload == "transformer_large" and args.global_batch == 0:
        # the four smaller benchmark configs, a few timed steps each (L2 flushed before every step)
        side = {}
        for name in ("mlp", "cnn", "lstm", "transformer_small"):
            w = dict(WORKLOADS[name])
            q = run_workload(torch, None, dev, w, 0, 1, local, 5, 3, e2e=True)
            qf = q["prof"]
            ach = qf["gemm_flops"] / (qf["gemm_ms"] / 1e3) / 1e12 if qf["gemm_ms"] > 0 else 0.0
            side[name] = {"global_batch": q["GB"], "ms_per_step": q["ms_total"] / 5, "samples_per_s": q["GB"] * 5 / (q["ms_total"] / 1e3),
                          "e2e_samples_per_s": q["e2e"]["value"], "launches_per_step": q["launches"] // 5,
                          "issued_contraction_flops_per_step": qf["gemm_flops"], "contraction_ms_per_step": qf["gemm_ms"],
                          "contraction_tflops": ach, "contraction_frac_of_bf16_sustained": ach / pk["bf16_tflops_sustained"],
                          "step_flops_over_step_time_tflops": qf["gemm_flops"] / (q["ms_total"] / 5 / 1e3) / 1e12, "loss": q["loss"]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, sample = cpu_baseline(workload, threads)
        cpu = {"value": v, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": "train samples/s (fwd+bwd+Adam)", "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload["name"], "global_batch": GB, "per_gpu_batch": r["B"], "params": r["params"],
                       "parallelism": f"dp{world}",
                       "l2": "L2 flushed (256 MB write) before every timed step, steps timed one by one" if r["flush"]
                       else "per-step working set (tens of GB) exceeds L2; no flush needed",
                       "semantics": "reference-literal (worker layout W=1)"},
            "loss": r["loss"], "clocks": r["clocks"], "gpu_launches": r["launches"], "roofline": roofline, "e2e": r["e2e"], "cpu_baseline": cpu,
        }
        if side is not None:
            line["configs"] = side
        print(json.dumps(line))
    if dist:
        dist.destroy_process_group()
    dev.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
