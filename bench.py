#!/usr/bin/env python
"""Throughput of the EmbeddingBag gather-and-pool path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c3|c5|rowshard] [--exchange nccl|push]

One "step" is one pooled call over one synthetic batch.  Rank 0 prints ONE JSON line.

N = 1   workload c2: table 1,000,000 x 128 fp16, 16384 bags, bag lengths Poisson(40)
        clipped to [1,200], Zipf(1.05) indices, mean pooling.  `value` times K back-to-back
        kernel launches over 8 rotating index batches resident in HBM; `e2e` times the same
        calls through the host-buffer session (pinned host inputs copied in, result copied
        out, every step); `roofline` is algorithmic bytes over the mean per-launch time;
        `cpu_baseline` is torch CPU EmbeddingBag on the same batch on this host's cores.
N > 1   workload rowshard (launched under torchrun, one rank per GPU): the c2 shape grown
        with N — a table of N x 1,000,000 rows split by rows, rank r holding rows
        [r*1e6, (r+1)*1e6), a global batch of N x 16384 bags that every rank scans, each
        rank pooling the rows it owns into fp32 partial bags, partials combined by
        reduce-scatter over NVLink (weak scaling: per-rank rows and per-rank lookups fixed).
--impl reference   times torch CPU EmbeddingBag (the ground truth of the reference's own
        unit test and the CPU baseline the metric names) on the same workload, on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NUM_BATCHES = 8
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the pooling kernel, from the ncu
# captures summarised under profiles/ (None where no capture of that workload exists yet).
NCU_DRAM_BYTES_PER_LAUNCH = {"c2": 35.9e6, "rowshard": None}
C2 = dict(rows=1_000_000, dim=128, bags=16384)


# ---- clocks --------------------------------------------------------------------------

class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _names(self, mask: int):
        nv = self.nv
        table = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        return {k for k, bit in table.items() if mask & bit}

    def _poll(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                self.reasons |= self._names(
                    self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception:
                break
            time.sleep(0.0005)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
        return {
            "sm_mhz": float(np.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ---- workload construction -------------------------------------------------------------

def make_batches(total_rows: int, total_bags: int, seed: int):
    from forward_b200 import workloads
    rng = np.random.default_rng(seed)
    sampler = workloads.ZipfSampler(total_rows, 1.05, rng)
    return [workloads.config2_bags(num_rows=total_rows, num_bags=total_bags, sampler=sampler,
                                   rng=rng) for _ in range(NUM_BATCHES)]


def algorithmic_bytes(bags, dim, gathered, out_itemsize, table_itemsize=2):
    from forward_b200 import workloads
    return workloads.algorithmic_bytes(
        gathered_rows=gathered, dim=dim, table_itemsize=table_itemsize,
        num_indices=bags.num_indices, num_offsets=bags.num_bags, index_itemsize=4,
        num_bags=bags.num_bags, out_itemsize=out_itemsize)


# ---- CPU arms ----------------------------------------------------------------------------

def cpu_embedding_bag_rate(table_np, batches, budget_s: float, min_reps: int = 3):
    """torch CPU EmbeddingBag (mean, fp16 table) on whole batches; lookups per second."""
    import torch

    from oracle import eb_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t = torch.from_numpy(table_np)
    prepared = [(torch.from_numpy(b.indices.astype(np.int64)),
                 torch.from_numpy(b.offsets.astype(np.int64)), b.num_indices) for b in batches]
    import torch.nn.functional as F
    for i, o, _ in prepared[:2]:
        F.embedding_bag(i, t, o, mode="mean")
    assert O.MODE_MEAN == 1
    done, lookups, reps = 0.0, 0, 0
    while reps < min_reps or done < budget_s:
        i, o, n = prepared[reps % len(prepared)]
        t0 = time.perf_counter()
        F.embedding_bag(i, t, o, mode="mean")
        done += time.perf_counter() - t0
        lookups += n
        reps += 1
    return lookups / done, cores, reps, done


def host_table(rows: int, dim: int, row_lo: int = 0):
    """The counter-generated table on the host (same bits as the device fill)."""
    from oracle import eb_oracle as O
    out = np.empty((rows, dim), dtype=np.float16)
    step = 1 << 16
    for lo in range(0, rows, step):
        n = min(step, rows - lo)
        out[lo:lo + n] = O.table_rows(np.arange(lo, lo + n, dtype=np.int64) + row_lo, dim, seed=1,
                                      scale=0.1, dtype=np.float16)
    return out


def run_reference(args, world: int, rank: int):
    if rank != 0:
        return
    total_rows, total_bags = C2["rows"] * world, C2["bags"] * world
    batches = make_batches(total_rows, total_bags, seed=1)
    import torch
    table = host_table(total_rows, C2["dim"])
    import torch.nn.functional as F
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t = torch.from_numpy(table)
    prepared = [(torch.from_numpy(b.indices.astype(np.int64)),
                 torch.from_numpy(b.offsets.astype(np.int64)), b.num_indices) for b in batches]
    for k in range(args.warmup):
        i, o, _ = prepared[k % NUM_BATCHES]
        F.embedding_bag(i, t, o, mode="mean")
    lookups = 0
    t0 = time.perf_counter()
    for k in range(args.steps):
        i, o, n = prepared[k % NUM_BATCHES]
        F.embedding_bag(i, t, o, mode="mean")
        lookups += n
    dt = time.perf_counter() - t0
    value = lookups / dt
    line = {
        "impl": "reference", "metric": "pooled_lookups_per_sec", "value": value,
        "unit": "lookups/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(world),
        "cpu_baseline": {"value": value, "unit": "lookups/s", "cores": cores, "kind": "port",
                         "sample": "torch CPU EmbeddingBag (mean, fp16 table), whole batches, "
                                   f"{args.steps} steps"},
        "e2e": {"value": value, "unit": "lookups/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(world: int):
    if world == 1:
        return {"workload": "c2: EmbeddingBag mean, table 1000000x128 fp16, 16384 bags/step, "
                            "lengths Poisson(40) clipped [1,200], Zipf(1.05) indices",
                "bags_per_step": C2["bags"], "table_rows": C2["rows"], "dim": C2["dim"],
                "l2_policy": "no flush: 256 MB table (> 126 MB L2) and 8 rotating index batches",
                "parallelism": "single"}
    return {"workload": f"rowshard: c2 shape grown x{world}: table {world}x1000000x128 fp16 split "
                        f"by rows, {world}x16384 bags/step scanned by every rank, partial bags "
                        "pushed to their owner ranks over NVLink and folded there",
            "bags_per_step": C2["bags"] * world, "table_rows": C2["rows"] * world,
            "dim": C2["dim"],
            "l2_policy": "no flush: 256 MB table shard per GPU (> 126 MB L2), 8 rotating batches",
            "parallelism": f"rowshard{world}"}


# ---- GPU arm ------------------------------------------------------------------------------

def run_ours(args, world: int, rank: int, local_rank: int):
    import torch

    from forward_b200 import capi
    from forward_b200 import dist as fd
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the package has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    sharded = world > 1
    if sharded:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    dim = C2["dim"]
    rows_local = C2["rows"]
    row_lo = rank * rows_local
    total_rows, total_bags = rows_local * world, C2["bags"] * world
    batches = make_batches(total_rows, total_bags, seed=1)
    table = torch.empty((rows_local, dim), dtype=torch.float16, device=dev)
    capi.fill_table(table, row_lo, seed=1, scale=0.1)
    d_batches = [(torch.from_numpy(b.indices).to(dev), torch.from_numpy(b.offsets).to(dev))
                 for b in batches]
    lookups_global = [b.num_indices for b in batches]
    gathered_local = [int(np.count_nonzero((b.indices >= row_lo) & (b.indices < row_lo + rows_local)))
                      for b in batches]
    stream = torch.cuda.current_stream()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps)]

    if sharded:
        wire = capi.F16 if args.wire == "f16" else capi.F32
        bag = fd.RowShardedBag(table, row_lo, mode=capi.MODE_MEAN, max_bags=total_bags,
                               exchange=args.exchange, wire_dtype=wire)
        local_out = torch.empty((total_bags, dim), dtype=torch.float32, device=dev)
        local_params = [capi.make_params(table, i, o, out=local_out, mode=capi.MODE_MEAN, row_lo=row_lo)
                        for i, o in d_batches]

        def step(k: int, timed: bool = False):
            i, o = d_batches[k % NUM_BATCHES]
            bag.forward(i, o, pool_events=(ev[2 * k], ev[2 * k + 1]) if timed else None)
    else:
        out = torch.empty((total_bags, dim), dtype=torch.float16, device=dev)
        params = [capi.make_params(table, i, o, out=out, mode=capi.MODE_MEAN) for i, o in d_batches]

        def step(k: int, timed: bool = False):
            if timed:
                ev[2 * k].record()
            capi.forward(params[k % NUM_BATCHES], stream.cuda_stream)
            if timed:
                ev[2 * k + 1].record()

    def barrier():
        if sharded:
            dist.barrier()
        torch.cuda.synchronize()

    # bring clocks up before the counted warm-up; a fixed count when ranks must stay in step
    if sharded:
        for k in range(int(args.preheat_ms * 5)):      # ~80 us a step: about the same duration
            step(k)
            if k % 64 == 63:
                torch.cuda.synchronize()
    else:
        t_end = time.perf_counter() + args.preheat_ms * 1e-3
        k = 0
        while time.perf_counter() < t_end:
            step(k)
            k += 1
            if k % 64 == 0:
                torch.cuda.synchronize()
    pool_only_us = None
    if sharded:
        # the same pooling without any exchange, for the overhead figure
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for k in range(20):
            capi.forward(local_params[k % NUM_BATCHES], stream.cuda_stream)
        n_po = max(20, min(args.steps, 200))
        a.record()
        for k in range(n_po):
            capi.forward(local_params[k % NUM_BATCHES], stream.cuda_stream)
        b.record()
        torch.cuda.synchronize()
        pool_only_us = a.elapsed_time(b) * 1e3 / n_po
    for k in range(args.warmup):
        step(k)
    barrier()

    sampler = ClockSampler(local_rank)
    launches0 = capi.lib().fwd_eb_launch_count()
    t_begin, t_finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    t_begin.record()
    for k in range(args.steps):
        step(k, timed=True)
    t_finish.record()
    barrier()
    clocks = sampler.stop()
    launches = capi.lib().fwd_eb_launch_count() - launches0
    total_ms = t_begin.elapsed_time(t_finish)
    kernel_ms = np.array([ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(args.steps)])
    exchange = None
    if sharded:
        if bag.check_status() != 0:
            raise RuntimeError("a bounded flag wait gave up during the timed region")
        tt = torch.tensor([total_ms, pool_only_us], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms, pool_only_us = float(tt[0].item()), float(tt[1].item())
        step_us = total_ms * 1e3 / args.steps
        wire_bytes = 2 if (args.exchange == "push" and args.wire == "f16") else 4
        egress = C2["bags"] * (world - 1) * dim * wire_bytes      # per rank per step
        exchange = {"method": args.exchange, "wire": args.wire if args.exchange == "push" else "f32",
                    "pool_only_us": pool_only_us, "step_us": step_us,
                    "overhead_frac": (step_us - pool_only_us) / pool_only_us,
                    "nvlink_egress_bytes_per_rank": egress,
                    "nvlink_floor_us_at_770GBs": egress / 770e9 * 1e6}
    lookups = sum(lookups_global[k % NUM_BATCHES] for k in range(args.steps))
    value = lookups / (total_ms * 1e-3)

    # roofline of the pooling kernel on this rank
    out_item = (2 if (sharded and args.exchange == "push" and args.wire == "f16") else 4) if sharded else 2
    alg = np.mean([algorithmic_bytes(batches[k % NUM_BATCHES], dim, gathered_local[k % NUM_BATCHES],
                                     out_item) for k in range(args.steps)])
    peak, peak_kind = measured_peak()
    achieved = alg / (kernel_ms.mean() * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get("rowshard" if sharded else "c2"),
                "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0,
                "kernel_us_mean": float(kernel_ms.mean() * 1e3),
                "kernel_us_median": float(np.median(kernel_ms) * 1e3),
                "algorithmic_bytes_per_launch": float(alg)}

    e2e = None
    cpu = None
    if not args.no_e2e:
        e2e = run_e2e_sharded(args, batches, bag, rank, world, dev) if sharded else \
            run_e2e(args, batches, table)
    if rank == 0 and not sharded and not args.no_cpu_baseline:
        tab = host_table(rows_local, dim)
        rate, cores, reps, secs = cpu_embedding_bag_rate(tab, batches, budget_s=args.cpu_seconds)
        cpu = {"value": rate, "unit": "lookups/s", "cores": cores, "kind": "port",
               "sample": f"torch CPU EmbeddingBag (mean, fp16 table) on whole c2 batches: {reps} "
                         f"calls, {secs:.1f} s"}

    if rank == 0:
        line = {
            "metric": "pooled_lookups_per_sec", "value": value, "unit": "lookups/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(world), "roofline": roofline, "cpu_baseline": cpu,
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        if exchange:
            line["exchange"] = exchange
        print(json.dumps(line), flush=True)
    if sharded:
        bag.close()
        dist.destroy_process_group()


def run_e2e_sharded(args, batches, bag, rank, world, dev):
    """N > 1: every step copies the whole batch from pinned host memory to this rank's GPU, runs
    the sharded call and copies this rank's slice of the result back to pinned memory."""
    import torch
    import torch.distributed as dist
    host = [(torch.from_numpy(b.indices).pin_memory(), torch.from_numpy(b.offsets).pin_memory())
            for b in batches]
    d_idx = [torch.empty_like(i, device=dev) for i, _ in host]
    d_off = [torch.empty_like(o, device=dev) for _, o in host]
    per = C2["bags"]
    h_out = [torch.empty((per, C2["dim"]), dtype=torch.float32).pin_memory() for _ in range(NUM_BATCHES)]

    def step(k):
        j = k % NUM_BATCHES
        d_idx[j].copy_(host[j][0], non_blocking=True)
        d_off[j].copy_(host[j][1], non_blocking=True)
        res = bag.forward(d_idx[j], d_off[j])
        h_out[j][:res.shape[0]].copy_(res, non_blocking=True)

    for k in range(max(args.warmup, 3)):
        step(k)
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for k in range(args.steps):
        step(k)
    torch.cuda.synchronize()
    dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    dt = float(dt.item())
    lookups = sum(batches[k % NUM_BATCHES].num_indices for k in range(args.steps))
    h2d = int(np.mean([b.num_indices * 4 + b.num_bags * 4 for b in batches]))
    return {"value": lookups / dt, "unit": "lookups/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": per * C2["dim"] * 4, "ms_per_step": dt / args.steps * 1e3,
            "note": "bytes are per rank; every rank receives the whole batch",
            "api": "forward_b200.dist.RowShardedBag.forward"}


def run_e2e(args, batches, table):
    """Same calls through the host-buffer session: pinned inputs in, result out, each step."""
    import torch

    from forward_b200 import capi
    from forward_b200.session import Session
    depth = 4
    max_n = max(b.num_indices for b in batches)
    s = Session(table_dtype=capi.F16, dim=C2["dim"], num_rows=C2["rows"], mode=capi.MODE_MEAN,
                max_indices=max_n, max_bags=C2["bags"], depth=depth, external_table=True)
    s.adopt_table(table.data_ptr())
    views = [s.slot(k) for k in range(depth)]
    sizes = []
    for k in range(depth):       # slot k carries batch k; its copy-in still happens every step
        b = batches[k % NUM_BATCHES]
        views[k][0][:b.num_indices] = b.indices
        views[k][1][:b.num_bags] = b.offsets
        sizes.append((b.num_indices, b.num_bags))
    h2d, d2h = s.copy_bytes(*sizes[0])
    steps = args.steps
    for k in range(max(args.warmup, depth)):
        s.wait(k % depth)
        s.submit(k % depth, *sizes[k % depth])
    for k in range(depth):
        s.wait(k)
    torch.cuda.synchronize()
    checksum = 0.0
    t0 = time.perf_counter()
    for k in range(steps):
        sl = k % depth
        s.wait(sl)                       # result of the call issued `depth` steps ago
        checksum += float(views[sl][3][0, 0])   # touch the returned result
        s.submit(sl, *sizes[sl])
    for k in range(depth):
        s.wait(k)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    lookups = sum(sizes[k % depth][0] for k in range(steps))
    s.close()
    return {"value": lookups / dt, "unit": "lookups/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "ms_per_step": dt / steps * 1e3,
            "calls_in_flight": depth, "api": "fwd_eb_session_submit / fwd_eb_session_wait"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--exchange", default="push", choices=["push", "a2a", "nccl"],
                    help="N>1: how partial bags reach their owners")
    ap.add_argument("--wire", default="f32", choices=["f32", "f16"],
                    help="N>1 with --exchange push: element type of the partials on NVLink")
    ap.add_argument("--preheat-ms", type=float, default=400.0,
                    help="untimed launches before the counted warm-up, to bring clocks up")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run "
                             "(--nproc-per-node N)")
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    run_ours(args, world, rank, local_rank)


if __name__ == "__main__":
    main()
