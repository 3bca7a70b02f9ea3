#!/usr/bin/env python
"""Throughput of the EmbeddingBag gather-and-pool path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload auto|c2|c2u|tablewise|rowshard|c5|c3|c4]
                    [--exchange auto|compact|push|stage|a2a|nccl] [--wire f32|f16] [--streams 1|2]
                    [--regions R] [--lookback EVERY,DEPTH] [--c4-replicate-mb M] [--local-streams 0|1|2]

One "step" is one pooled call over one synthetic batch.  Rank 0 prints ONE JSON line.

Workloads (all synthetic: shapes and distributions only, rotating index batches per table)
  c2         N = 1.  Table 1,000,000 x 128 fp16, 16384 bags, lengths Poisson(40) clipped to
             [1,200], Zipf(1.05) indices, mean pooling, fp16 output.
  tablewise  N > 1 (launch under torchrun, one rank per GPU).  The c2 family grown with N: N
             tables of the c2 shape, one per GPU, each looked up by its own c2 batch of 16384
             bags; every rank pools its table for the whole batch and the pooled rows are
             exchanged so that rank g ends with [16384/N, N, 128] (the all-to-all of pooled
             outputs of table-wise placement).  Weak scaling: one table and one batch per GPU.
  rowshard   N > 1.  ONE table of N x 1,000,000 rows split by rows, N x 16384 bags per step that
             every rank scans; partial bags go to their owner ranks and are folded there.
  c5         N >= 1.  Table 1,000,000,000 x 64 fp16 (128 GB) split by rows over N GPUs, 131072
             bags of 1..100 uniform indices, sum.  Strong scaling.
  c3         N = 1.  Table 4,000,000 x 256 fp16, 8192 bags of 0..64 uniform indices, 5 % of the
             indices are padding_idx 0, max pooling.
  c4         N >= 1.  26 tables of 1e3..3e7 rows x 128 fp32 (42 GB in all), 65536 bags of exactly
             20 Zipf(1.1) indices per table with per-sample weights, sum.  Tables under
             --c4-replicate-mb MiB (default 256: 18 of the 26) live on every rank, which pools
             its own bags of them; the others are placed whole on one rank each (greedy by
             lookups, then bytes), pooled there for the whole batch, and their rows go to
             [65536/N, 26, 128] fp32 on the rank owning the bag.  Strong scaling; N = 1 holds
             all 26 tables and pools them with fwd_eb_forward_many.
  auto       c2 at N = 1, tablewise at N > 1.

`value` times K steps on data resident in HBM (CUDA events, barrier + synchronize on both sides,
max over ranks; the median of --regions such regions).  Steps are independent batches and, with
--streams 2 (the default), alternate over two CUDA streams per GPU, each with its own output and
scratch, so that one step's grid runs beside the tail of the step before; --streams 1 queues every
step on one stream (`roofline.kernel_us_one_stream` carries that figure in the default line too); `roofline` is the pooling kernel's algorithmic bytes over its mean event time;
`e2e` repeats the steps with inputs copied from pinned host memory and results copied back every
step; `cpu_baseline` / `--impl reference` time torch CPU EmbeddingBag (the ground truth of the
reference's own unit test and the CPU baseline the metric names) on the same workload.
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
NCU_TRAFFIC_FILE = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
C2 = dict(rows=1_000_000, dim=128, bags=16384)
C5 = dict(rows=1_000_000_000, dim=64, bags=131072)
C3 = dict(rows=4_000_000, dim=256, bags=8192)
C4 = dict(tables=26, dim=128, bags=65536, pooling=20, cpu_row_cap=1 << 19)


# ---- clocks --------------------------------------------------------------------------

class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.0005):
        self.period_s = period_s
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
            time.sleep(self.period_s)

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


def ncu_traffic(workload: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's pooling kernel, as
    the last committed ncu capture measured it (profiles/ncu_dram_traffic.json names the capture
    and the source revision it was taken on); (None, None) where no capture of that workload exists."""
    try:
        with open(NCU_TRAFFIC_FILE) as f:
            entry = json.load(f)["workloads"].get(workload)
        if entry:
            return float(entry["dram_bytes_per_launch"]), f"{entry['capture']} @ {entry['revision']}"
    except Exception:
        pass
    return None, None


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ---- workload construction -------------------------------------------------------------

def resolve_workload(name: str, world: int) -> str:
    if name == "auto":
        return "c2" if world == 1 else "tablewise"
    if name in ("c2", "c2u", "c3") and world != 1:
        raise SystemExit(f"workload {name} is a single-GPU workload")
    if name in ("tablewise", "rowshard") and world == 1:
        raise SystemExit(f"workload {name} needs more than one GPU (launch under torchrun)")
    return name


def c2_batches(total_rows: int, total_bags: int, seed: int):
    from forward_b200 import workloads
    rng = np.random.default_rng(seed)
    sampler = workloads.ZipfSampler(total_rows, 1.05, rng)
    return [workloads.config2_bags(num_rows=total_rows, num_bags=total_bags, sampler=sampler,
                                   rng=rng) for _ in range(NUM_BATCHES)]


def make_batches(workload: str, world: int, table_id: int = 0):
    """The batches one table sees.  Every rank draws the same batches for a shared table."""
    from forward_b200 import workloads
    if workload == "c2":
        return c2_batches(C2["rows"], C2["bags"], seed=1)
    if workload == "c2u":     # c2's shape and bag lengths, uniform indices: no cache help
        rng = np.random.default_rng(11)
        return [workloads.ragged_bags(C2["rows"], np.clip(rng.poisson(40.0, C2["bags"]), 1, 200), rng)
                for _ in range(NUM_BATCHES)]
    if workload == "tablewise":
        return c2_batches(C2["rows"], C2["bags"], seed=1 + 7919 * table_id)
    if workload == "rowshard":
        return c2_batches(C2["rows"] * world, C2["bags"] * world, seed=1)
    if workload == "c5":
        return [workloads.config5_bags(seed=4 + b, num_rows=C5["rows"]) for b in range(4)]
    if workload == "c3":
        return [workloads.config3_bags(seed=2 + b) for b in range(NUM_BATCHES)]
    raise ValueError(workload)


def table_seed(workload: str, table_id: int) -> tuple[int, float]:
    """(seed, scale) of the counter-generated table."""
    if workload in ("c2", "c2u", "tablewise"):
        return 1 + table_id, 0.1
    if workload == "rowshard":
        return 1, 0.1
    if workload == "c5":
        return 4, 0.05
    return 2, 0.1


def describe(workload: str, world: int, args):
    base = {"l2_policy": "no flush: table (shard) larger than the 126 MB L2 and rotating index "
                         "batches; skewed laws keep their hot rows cached, which is a property "
                         "of the workload"}
    if world > 1 and workload != "c4" and int(getattr(args, "streams", 1) or 1) > 1:
        base["streams"] = ("consecutive steps (independent batches) alternate over 2 CUDA streams per rank; flags, "
                           "waits and folds stay in step order on the pipeline's side stream")
    if world == 1 and workload != "c4" and int(getattr(args, "streams", 1) or 1) > 1:
        base["streams"] = (f"consecutive steps (independent batches) rotate over {int(args.streams)} CUDA streams, "
                           "each with its own output buffer; the timed region forks them behind its start "
                           "event and joins them before its end event")
    if workload == "c2":
        base.update(workload="c2: EmbeddingBag mean, table 1000000x128 fp16, 16384 bags/step, lengths "
                             "Poisson(40) clipped [1,200], Zipf(1.05) indices",
                    bags_per_step=C2["bags"], table_rows=C2["rows"], dim=C2["dim"], parallelism="single")
    elif workload == "c2u":
        base.update(workload="c2u: the c2 shape (table 1000000x128 fp16, 16384 bags/step, lengths Poisson(40) "
                             "clipped [1,200], mean) with UNIFORM indices: the HBM-bound variant",
                    bags_per_step=C2["bags"], table_rows=C2["rows"], dim=C2["dim"], parallelism="single")
    elif workload == "tablewise":
        base.update(workload=f"tablewise: {world} tables of the c2 shape (1000000x128 fp16, mean), one "
                             f"per GPU, each with its own 16384-bag c2 batch per step; pooled rows "
                             f"exchanged to [16384/{world}, {world}, 128] per rank",
                    bags_per_step=C2["bags"] * world, table_rows=C2["rows"] * world, dim=C2["dim"],
                    parallelism=f"tablewise{world}", exchange=args.exchange)
    elif workload == "rowshard":
        base.update(workload=f"rowshard: one table {world}x1000000x128 fp16 split by rows, {world}x16384 "
                             "bags/step scanned by every rank, partial bags folded at their owners",
                    bags_per_step=C2["bags"] * world, table_rows=C2["rows"] * world, dim=C2["dim"],
                    parallelism=f"rowshard{world}", exchange=args.exchange, wire=args.wire)
    elif workload == "c5":
        window = f"; this GPU holds 1 of {args.c5_window} row windows and pools its partial bags only" \
            if (world == 1 and getattr(args, "c5_window", 1) > 1) else ""
        base.update(workload=f"c5: EmbeddingBag sum, table {C5['rows']}x64 fp16 "
                             f"({C5['rows'] * 128 / 1e9:.0f} GB) split by rows, "
                             "131072 bags/step of 1..100 uniform indices" + window,
                    bags_per_step=C5["bags"], table_rows=C5["rows"], dim=C5["dim"],
                    parallelism=f"rowshard{world}" if world > 1 else "single",
                    exchange=args.exchange if world > 1 else None, wire=args.wire)
    elif workload == "c4":
        capped = f" [tables cut to {args.c4_max_rows} rows: a profiler-sized case]" \
            if getattr(args, "c4_max_rows", 0) else ""
        mb = int(getattr(args, "c4_replicate_mb", 0)) if world > 1 else 0
        if mb:
            from forward_b200 import workloads
            small = sum(1 for r in workloads.config4_rows() if int(r) * C4["dim"] * 4 < (mb << 20))
            placing = (f"the {small} tables under {mb} MiB live on every rank, which pools its own bags of "
                       f"them; the other {C4['tables'] - small} are placed whole on one rank each and their ")
        else:
            placing = "tables placed whole on ranks, "
        base.update(workload="c4: 26 tables of 1e3..3e7 rows x 128 fp32 (42 GB), 65536 bags x 20 Zipf(1.1) "
                             "indices per table, per-sample weights, sum; " + placing +
                             f"pooled rows exchanged to [65536/{world}, 26, 128] fp32 per rank" + capped,
                    replicated_below_mib=mb,
                    bags_per_step=C4["bags"], tables=C4["tables"], dim=C4["dim"],
                    parallelism=f"tablewise{world}" if world > 1 else "single",
                    exchange=args.exchange if world > 1 else None,
                    l2_policy="no flush: one step reads 18 GB of rows from 42 GB of tables")
    elif workload == "c3":
        base.update(workload="c3: EmbeddingBag max, table 4000000x256 fp16, 8192 bags/step of 0..64 "
                             "uniform indices, 5% padding_idx=0",
                    bags_per_step=C3["bags"], table_rows=C3["rows"], dim=C3["dim"], parallelism="single")
    return base


def compute_dtype(workload: str) -> str:
    """The arithmetic type of the pooling: sums and means accumulate in fp32 whatever the table
    holds; max over fp16 rows compares in fp16 and carries the winner's bits."""
    return "f16" if workload == "c3" else "f32"


def scaling_kind(workload: str) -> str:
    return "strong" if workload in ("c5", "c4") else "weak"


# ---- CPU arms ----------------------------------------------------------------------------

def host_table(rows: int, dim: int, row_lo: int, seed: int, scale: float):
    """The counter-generated table on the host (same bits as the device fill)."""
    from oracle import eb_oracle as O
    out = np.empty((rows, dim), dtype=np.float16)
    step = 1 << 16
    for lo in range(0, rows, step):
        n = min(step, rows - lo)
        out[lo:lo + n] = O.table_rows(np.arange(lo, lo + n, dtype=np.int64) + row_lo, dim, seed=seed,
                                      scale=scale, dtype=np.float16)
    return out


class CpuWorkload:
    """torch CPU EmbeddingBag over the same tables and batches; one call of `step` = one bench
    step (all tables).  A table too large for host memory is replaced by a 2**27-row stand-in
    with the indices folded into it (same lookups; said so in `sample`)."""

    def __init__(self, workload: str, world: int):
        import torch
        import torch.nn.functional as F
        self.F = F
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.note = ""
        self.mode, self.pad = "mean", None
        if workload in ("c2", "c2u", "tablewise"):
            n_tab = 1 if workload != "tablewise" else world
            self.tables = [torch.from_numpy(host_table(C2["rows"], C2["dim"], 0, *table_seed(workload, t)))
                           for t in range(n_tab)]
            self.batches = [make_batches(workload, world, t) for t in range(n_tab)]
        elif workload == "rowshard":
            self.tables = [torch.from_numpy(host_table(C2["rows"] * world, C2["dim"], 0, 1, 0.1))]
            self.batches = [make_batches(workload, world)]
        elif workload == "c5":
            rows = 1 << 27
            self.tables = [torch.from_numpy(host_table(rows, C5["dim"], 0, 4, 0.05))]
            bs = make_batches(workload, world)
            for b in bs:
                b.indices %= rows
            self.batches = [bs]
            self.mode = "sum"
            self.note = " (table cut to 2^27 rows, indices folded into it: same lookups)"
        elif workload == "c3":
            self.tables = [torch.from_numpy(host_table(C3["rows"], C3["dim"], 0, 2, 0.1))]
            self.batches = [make_batches(workload, world)]
            self.mode, self.pad = "max", 0
        elif workload == "c4":
            from forward_b200 import workloads
            cap = C4["cpu_row_cap"]
            self.mode = "sum"
            self.tables, self.batches, self.prepared = [], [], []
            for t, rows in enumerate(workloads.config4_rows()):
                held = int(min(rows, cap))
                # values do not affect timing: a plain normal draw instead of the counter generator
                self.tables.append(torch.empty((held, C4["dim"]), dtype=torch.float32).normal_(0, 0.1))
                b = workloads.config4_bags(t, int(rows))
                self.batches.append([b])
                i = torch.from_numpy((b.indices % held).astype(np.int64)).view(-1, C4["pooling"])
                w = torch.from_numpy(b.per_sample_weights).view(-1, C4["pooling"])
                self.prepared.append([(i, None, w)])
            self.note = f" (tables above {cap} rows cut to {cap} rows, indices folded: same lookups)"
            return
        self.prepared = [[(torch.from_numpy(b.indices.astype(np.int64)),
                           torch.from_numpy(b.offsets.astype(np.int64)), None) for b in bs]
                         for bs in self.batches]

    def step(self, k: int) -> int:
        done = 0
        for t, table in enumerate(self.tables):
            nb = len(self.prepared[t])
            i, o, w = self.prepared[t][k % nb]
            self.F.embedding_bag(i, table, o, mode=self.mode, padding_idx=self.pad,
                                 per_sample_weights=w)
            done += self.batches[t][k % nb].num_indices
        return done


def host_info() -> dict:
    """CPU model string and torch version, for the CPU-arm lines."""
    import torch
    model = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    model = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    return {"cpu_model": model, "torch": torch.__version__}


def cpu_baseline(workload: str, world: int, budget_s: float):
    cw = CpuWorkload(workload, world)
    for k in range(2):
        cw.step(k)
    secs, lookups, reps = 0.0, 0, 0
    while reps < 3 or secs < budget_s:
        t0 = time.perf_counter()
        n = cw.step(reps)
        secs += time.perf_counter() - t0
        lookups += n
        reps += 1
    return {"value": lookups / secs, "unit": "lookups/s", "cores": cw.cores, "kind": "port",
            "sample": f"torch CPU EmbeddingBag on whole {workload} steps{cw.note}: {reps} steps, "
                      f"{secs:.1f} s", **host_info()}


def run_reference(args, world: int, rank: int):
    if rank != 0:
        return
    workload = resolve_workload(args.workload, world)
    if workload == "c4":       # a step is 34 M lookups (a quarter of a second of CPU time)
        args.steps, args.warmup = min(args.steps, 40), min(args.warmup, 3)
    cw = CpuWorkload(workload, world)
    for k in range(args.warmup):
        cw.step(k)
    lookups = 0
    t0 = time.perf_counter()
    for k in range(args.steps):
        lookups += cw.step(k)
    dt = time.perf_counter() - t0
    value = lookups / dt
    line = {
        "impl": "reference", "metric": "pooled_lookups_per_sec", "value": value,
        "unit": "lookups/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": scaling_kind(workload), "vs_baseline": None,
        "dtype": compute_dtype(workload), "table_dtype": "f32" if workload == "c4" else "f16",
        "data": "synthetic",
        "config": describe(workload, world, args),
        "cpu_baseline": {"value": value, "unit": "lookups/s", "cores": cw.cores, "kind": "port",
                         "sample": f"torch CPU EmbeddingBag on whole {workload} steps{cw.note}, "
                                   f"{args.steps} steps", **host_info()},
        "e2e": {"value": value, "unit": "lookups/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ------------------------------------------------------------------------------

class GpuWorkload:
    """Device-resident table, batches and the step closure of one workload on this rank."""

    def __init__(self, workload: str, world: int, rank: int, dev, args):
        import torch

        from forward_b200 import capi
        from forward_b200 import dist as fd
        self.workload, self.world, self.rank, self.dev, self.args = workload, world, rank, dev, args
        self.capi, self.fd, self.torch = capi, fd, torch
        self.bag = None
        self.pool_only = None
        self.resident = True      # the timed steps read device-resident batches; the e2e loop clears this
        self.out_itemsize = 2
        self.row_lo = 0
        local_filter = None
        if workload in ("c2", "c2u", "tablewise"):
            self.dim, rows, self.mode, self.pad = C2["dim"], C2["rows"], capi.MODE_MEAN, -1
            self.batches = make_batches(workload, world, rank)
        elif workload == "rowshard":
            self.dim, rows, self.mode, self.pad = C2["dim"], C2["rows"], capi.MODE_MEAN, -1
            self.row_lo = rank * rows
            self.batches = make_batches(workload, world)
            local_filter = (self.row_lo, self.row_lo + rows)
        elif workload == "c5":
            self.dim, self.mode, self.pad = C5["dim"], capi.MODE_SUM, -1
            self.row_lo, rows = fd.shard_rows(C5["rows"], world, rank)
            self.batches = make_batches(workload, world)
            local_filter = (self.row_lo, self.row_lo + rows) if world > 1 else None
            if world == 1 and args.c5_window > 1:
                # one GPU doing the pooling of ONE rank of a G-way row split (no exchange): the
                # per-rank kernel of the sharded runs, where ncu can look at it
                self.row_lo, rows = fd.shard_rows(C5["rows"], args.c5_window, args.c5_window // 2)
                local_filter = (self.row_lo, self.row_lo + rows)
        else:
            self.dim, rows, self.mode, self.pad = C3["dim"], C3["rows"], capi.MODE_MAX, 0
            self.batches = make_batches(workload, world)
        seed, scale = table_seed(workload, rank)
        self.table = torch.empty((rows, self.dim), dtype=torch.float16, device=dev)
        capi.fill_table(self.table, self.row_lo, seed=seed, scale=scale)
        self.nb = len(self.batches)
        self.d_batches = [(torch.from_numpy(b.indices).to(dev), torch.from_numpy(b.offsets).to(dev))
                          for b in self.batches]
        self.gathered = []
        for b in self.batches:
            keep = np.ones(b.num_indices, dtype=bool)
            if self.pad >= 0:
                keep &= b.indices != self.pad
            if local_filter:
                keep &= (b.indices >= local_filter[0]) & (b.indices < local_filter[1])
            self.gathered.append(int(np.count_nonzero(keep)))
        self._last = None
        self.local_filter = local_filter
        self._build_step()

    def _build_step(self):
        torch, capi, fd, args = self.torch, self.capi, self.fd, self.args
        dev = self.dev
        stream = torch.cuda.current_stream()
        bags_n = self.batches[0].num_bags
        if self.world == 1:
            # Consecutive steps are independent batches: they rotate over `lanes` streams (lane 0 is
            # the current stream), each lane with its own output and scratch, so that one step's grid
            # runs beside the tail of the step before (a grid of this size is under two waves, and on
            # one stream the next grid starts only when the last CTA of this one has finished).
            lanes = max(1, int(getattr(args, "streams", 1) or 1))
            self.lane_streams = [stream] + [torch.cuda.Stream() for _ in range(lanes - 1)]
            self._fork = torch.cuda.Event()
            self._joins = [torch.cuda.Event() for _ in range(lanes - 1)]
            outs = [torch.empty((bags_n, self.dim), dtype=torch.float16, device=dev) for _ in range(lanes)]
            self._outs = outs
            self._params = [[capi.make_params(self.table, i, o, out=out, mode=self.mode, padding_idx=self.pad,
                                              row_lo=self.row_lo) for i, o in self.d_batches] for out in outs]

            if self.local_filter:
                # one rank's share of a row-sharded table on one GPU: the two kernels a rank runs per
                # step (window compaction, pooling of the dense sub-bags), with local stores
                max_n = max(b.num_indices for b in self.batches)
                scratch = [(torch.empty(max_n, dtype=torch.int32, device=dev),
                            torch.empty((bags_n, 2), dtype=torch.int32, device=dev)) for _ in range(lanes)]
                cps = [capi.make_compacted_params(self.table, kept, bounds, out=out, mode=self.mode)
                       for (kept, bounds), out in zip(scratch, outs)]
                self._compact_keep = scratch

                def step(k, events=None, lane=None):
                    lane = 0 if events else (k % lanes if lane is None else lane)
                    st = self.lane_streams[lane]
                    kept, bounds = scratch[lane]
                    if events:
                        events[0].record()
                    capi.compact_window(self._params[lane][k % self.nb], kept, bounds, stream=st.cuda_stream)
                    capi.forward(cps[lane], st.cuda_stream)
                    if events:
                        events[1].record()
                    self._last = outs[lane]
                self.step = step
                return

            def step(k, events=None, lane=None):
                lane = 0 if events else (k % lanes if lane is None else lane)
                if events:
                    events[0].record()
                capi.forward(self._params[lane][k % self.nb], self.lane_streams[lane].cuda_stream)
                if events:
                    events[1].record()
                self._last = outs[lane]
            self.step = step
            return
        if self.workload == "tablewise":
            self.bag = fd.TableWiseBags({self.rank: self.table}, list(range(self.world)), dim=self.dim,
                                        max_bags=bags_n, exchange=args.exchange, wire_dtype=capi.F16,
                                        mode=self.mode, ship=args.ship, lookback=args.lookback,
                                        lanes=min(2, max(1, int(args.streams))))
            self.out_itemsize = 2 if args.exchange == "push" else 4

            self._prepared = [self.bag.prepare({self.rank: (i, o, None)}) for i, o in self.d_batches]

            def step(k, events=None):
                self._last = self.bag.forward(self._prepared[k % self.nb], pool_events=events,
                                               inputs_ready=self.resident)
        else:
            wire = capi.F16 if args.wire == "f16" else capi.F32
            max_n = max(b.num_indices for b in self.batches)
            self.bag = fd.RowShardedBag(self.table, self.row_lo, mode=self.mode, max_bags=bags_n,
                                        exchange=args.exchange, wire_dtype=wire, max_indices=max_n,
                                        ship=args.ship, lookback=args.lookback,
                                        lanes=min(2, max(1, int(args.streams))) if args.exchange in
                                        ("push", "stage", "compact") else 1)
            self.out_itemsize = 2 if (args.exchange in ("push", "stage", "compact") and args.wire == "f16") else 4

            self._prepared = [self.bag.prepare(i, o) for i, o in self.d_batches]

            def step(k, events=None):
                self._last = self.bag.forward(self._prepared[k % self.nb], pool_events=events,
                                               inputs_ready=self.resident)
        self.step = step
        # the same pooling without any exchange, for the overhead figure — queued as the steps are:
        # alternating over as many streams, each with its own output and scratch
        lanes = min(2, max(1, int(args.streams))) if (self.workload == "tablewise" or args.exchange in
                                                      ("push", "stage", "compact")) else 1
        self._po_streams = [stream] + [torch.cuda.Stream() for _ in range(lanes - 1)]
        self._po_fork = torch.cuda.Event()
        self._po_joins = [torch.cuda.Event() for _ in range(lanes - 1)]
        local_dtype = torch.float16 if self.workload == "tablewise" else torch.float32
        local_outs = [torch.empty((bags_n, self.dim), dtype=local_dtype, device=dev) for _ in range(lanes)]
        lps = [[capi.make_params(self.table, i, o, out=lo, mode=self.mode, padding_idx=self.pad,
                                 row_lo=self.row_lo) for i, o in self.d_batches] for lo in local_outs]
        if self.workload != "tablewise" and args.exchange == "compact":
            # the same two kernels as the step (window compaction, pooling of the dense sub-bags)
            # with local stores and no flags or fold
            max_n = max(b.num_indices for b in self.batches)
            wire_dt = torch.float16 if args.wire == "f16" else torch.float32
            scratch = [(torch.empty(max_n, dtype=torch.int32, device=dev),
                        torch.empty((bags_n, 2), dtype=torch.int32, device=dev),
                        torch.empty((bags_n, self.dim), dtype=wire_dt, device=dev)) for _ in range(lanes)]
            cps = [capi.make_compacted_params(self.table, kept, bounds, out=lw, mode=capi.MODE_SUM)
                   for kept, bounds, lw in scratch]
            self._po_keep = scratch

            def pool_only(k):
                lane = k % lanes
                st = self._po_streams[lane].cuda_stream
                capi.compact_window(lps[lane][k % self.nb], scratch[lane][0], scratch[lane][1], stream=st)
                capi.forward(cps[lane], st)
            self.pool_only = pool_only
        else:
            self.pool_only = lambda k: capi.forward(lps[k % lanes][k % self.nb],
                                                    self._po_streams[k % lanes].cuda_stream)

    def pool_fork(self):
        if len(self._po_streams) > 1:
            self._po_fork.record(self._po_streams[0])
            for st in self._po_streams[1:]:
                st.wait_event(self._po_fork)

    def pool_join(self):
        for st, ev in zip(self._po_streams[1:], self._po_joins):
            ev.record(st)
            self._po_streams[0].wait_event(ev)

    def fork(self):
        """The other lanes start where the current stream stands (call after the region's start event)."""
        lanes = getattr(self, "lane_streams", None)
        if lanes and len(lanes) > 1:
            self._fork.record(lanes[0])
            for st in lanes[1:]:
                st.wait_event(self._fork)

    def join(self):
        """The current stream waits for every lane (call before the region's end event)."""
        lanes = getattr(self, "lane_streams", None)
        if lanes and len(lanes) > 1:
            for st, ev in zip(lanes[1:], self._joins):
                ev.record(st)
                lanes[0].wait_event(ev)

    def set_device_batches(self, d_batches):
        """Point the step at other device copies of the same batches (the e2e loop's)."""
        self.d_batches = d_batches
        if self.world > 1:
            if self.workload == "tablewise":
                self._prepared = [self.bag.prepare({self.rank: (i, o, None)}) for i, o in d_batches]
            else:
                self._prepared = [self.bag.prepare(i, o) for i, o in d_batches]
        if self.world == 1:
            self._params = [[self.capi.make_params(self.table, i, o, out=out, mode=self.mode,
                                                   padding_idx=self.pad, row_lo=self.row_lo)
                             for i, o in d_batches] for out in self._outs]

    def result(self):
        return self._last

    def lookups(self, k: int) -> int:
        """Lookups of step k on the table this rank's batches address."""
        return self.batches[k % self.nb].num_indices

    def algorithmic_bytes(self, k: int) -> float:
        from forward_b200 import workloads
        b = self.batches[k % self.nb]
        return workloads.algorithmic_bytes(
            gathered_rows=self.gathered[k % self.nb], dim=self.dim, table_itemsize=2,
            num_indices=b.num_indices, num_offsets=b.num_bags, index_itemsize=4,
            num_bags=b.num_bags, out_itemsize=self.out_itemsize)


class C4Workload:
    """Config 4 on this rank: the tables placed here, their fixed-length weighted batches, and
    the step that pools every local table for the whole batch (N > 1: with the pooled rows
    pushed to the bags' owner ranks).  Same surface as GpuWorkload where run_ours() uses it."""

    workload = "c4"

    def __init__(self, world: int, rank: int, dev, args):
        import torch

        from forward_b200 import capi, workloads
        from forward_b200 import dist as fd
        self.world, self.rank, self.dev, self.args = world, rank, dev, args
        self.capi, self.torch = capi, torch
        self.dim, self.mode, self.pad = C4["dim"], capi.MODE_SUM, -1
        self.out_itemsize = 4
        self.L = C4["pooling"]
        cap = getattr(args, "c4_max_rows", 0) or 0
        self.rows = [int(min(r, cap)) if cap else int(r) for r in workloads.config4_rows()]
        self.T = len(self.rows)
        n_per_table = C4["bags"] * self.L
        self.owner = fd.place_tables([r * self.dim * 4 for r in self.rows], world,
                                     [n_per_table] * self.T,
                                     replicate_below_bytes=int(getattr(args, "c4_replicate_mb", 0)) << 20)
        self.mine = [t for t in range(self.T) if self.owner[t] == rank]
        # tables small enough to live on every rank: each rank pools its own bags of them, no exchange
        self.replicated = [t for t in range(self.T) if self.owner[t] == fd.REPLICATED]
        self.here = sorted(self.mine + self.replicated)
        per = fd.bags_per_rank(C4["bags"], world)
        self.own_lo = min(C4["bags"], rank * per)
        self.own_n = min(C4["bags"], (rank + 1) * per) - self.own_lo
        self.tables, self.bags, self.h_in, self.d_in, self.d_idx, self.d_w = {}, {}, {}, {}, {}, {}
        self.copies = []      # (device view, pinned host view) of what a step's inputs are on this rank
        for t in self.here:
            tab = torch.empty((self.rows[t], self.dim), dtype=torch.float32, device=dev)
            capi.fill_table(tab, 0, seed=300 + t, scale=0.1)
            self.tables[t] = tab
            b = workloads.config4_bags(t, self.rows[t])
            self.bags[t] = b
            # indices and weights of a table share one pinned block: one copy per table per step
            blk = np.concatenate([b.indices, b.per_sample_weights.view(np.int32)])
            self.h_in[t] = torch.from_numpy(blk).pin_memory()
            self.d_in[t] = self.h_in[t].to(dev)
            self.d_idx[t] = self.d_in[t][:n_per_table]
            self.d_w[t] = self.d_in[t][n_per_table:].view(torch.float32)
            if t in self.mine:
                self.copies.append((self.d_in[t], self.h_in[t]))
            else:             # a replicated table: only this rank's bags (their indices, their weights)
                a, b = self.own_lo * self.L, (self.own_lo + self.own_n) * self.L
                for base in (0, n_per_table):
                    self.copies.append((self.d_in[t][base + a:base + b], self.h_in[t][base + a:base + b]))
        self.batches = [workloads.Bags(np.empty(n_per_table, dtype=np.int32), None, fixed_len=self.L)]
        self.bag = None
        self.pool_only = None
        self._last = None
        stream = torch.cuda.current_stream()
        self.launches_per_step = len(self.here)
        if world == 1:
            out = torch.empty((C4["bags"], self.T, self.dim), dtype=torch.float32, device=dev)
            params = [capi.make_params(self.tables[t], self.d_idx[t], None, out=out[:, t, :],
                                       mode=self.mode, fixed_len=self.L,
                                       per_sample_weights=self.d_w[t]) for t in self.mine]

            packed = capi.pack_params(params)
            one_stream = getattr(args, "local_streams", None) == 0

            def step(k, events=None):
                if events:
                    events[0].record()
                if one_stream:
                    for p in params:
                        capi.forward(p, stream.cuda_stream)
                else:       # the 26 tables are independent: spread over the library's streams
                    capi.forward_many(packed, stream.cuda_stream)
                if events:
                    events[1].record()
                self._last = out
            self.step = step
            return
        self.bag = fd.TableWiseBags(self.tables, self.owner, dim=self.dim, max_bags=C4["bags"],
                                    exchange=args.exchange, wire_dtype=capi.F32, mode=self.mode,
                                    fixed_len=self.L, ship=args.ship, lookback=args.lookback,
                                    local_streams=getattr(args, "local_streams", None))
        prepared = self.bag.prepare({t: (self.d_idx[t], None, self.d_w[t]) for t in self.here})

        def step(k, events=None):
            self._last = self.bag.forward(prepared, pool_events=events)
        self.step = step
        local = torch.empty((C4["bags"], max(1, len(self.here)), self.dim), dtype=torch.float32,
                            device=dev)
        a, b = self.own_lo * self.L, (self.own_lo + self.own_n) * self.L
        lp = [capi.make_params(self.tables[t], self.d_idx[t], None, out=local[:, j, :], mode=self.mode,
                               fixed_len=self.L, per_sample_weights=self.d_w[t]) if t in self.mine else
              capi.make_params(self.tables[t], self.d_idx[t][a:b], None, out=local[:self.own_n, j, :],
                               mode=self.mode, fixed_len=self.L, per_sample_weights=self.d_w[t][a:b])
              for j, t in enumerate(self.here)]

        # the same launches with local stores only, queued as the step queues them: round robin over
        # the current stream and two more
        n_aux = 2 if getattr(args, "local_streams", None) is None else int(args.local_streams)
        order = [p for p, t in zip(lp, self.here) if t in self.mine] + \
                [p for p, t in zip(lp, self.here) if t not in self.mine]
        n_mine, shares = len(self.mine), len(self.replicated) > 0
        aux = [torch.cuda.Stream() for _ in range(min(n_aux, max(0, len(order) - 1)))]
        fork, joins = torch.cuda.Event(), [torch.cuda.Event() for _ in aux]

        def pool_only(k):
            if aux:
                fork.record(stream)
                for a_ in aux:
                    a_.wait_event(fork)
            for i, p in enumerate(order):
                if i < n_mine and shares:        # whole tables together, the shares beside them
                    lane = 0
                elif shares and n_mine:
                    lane = 1 + (i - n_mine) % len(aux) if aux else 0
                else:
                    lane = i % (len(aux) + 1)
                capi.forward(p, stream.cuda_stream if lane == 0 else aux[lane - 1].cuda_stream)
            for a_, j in zip(aux, joins):
                j.record(a_)
                stream.wait_event(j)
        self.pool_only = pool_only

    def result(self):
        return self._last

    def lookups(self, k: int) -> int:
        return (len(self.mine) * C4["bags"] + len(self.replicated) * self.own_n) * self.L

    def algorithmic_bytes(self, k: int) -> float:
        from forward_b200 import workloads
        total = 0.0
        for count, bags in ((len(self.mine), C4["bags"]), (len(self.replicated), self.own_n)):
            n = bags * self.L
            total += count * workloads.algorithmic_bytes(
                gathered_rows=n, dim=self.dim, table_itemsize=4, num_indices=n, num_offsets=0,
                index_itemsize=4, num_bags=bags, out_itemsize=4, weighted=True)
        return float(total)

    def egress_bytes(self) -> int:
        """Pooled bytes this rank sends to other ranks per step."""
        return len(self.mine) * C4["bags"] * (self.world - 1) // self.world * self.dim * 4

    def verify(self) -> bool:
        """A sample of the bags of EVERY rank, gathered to every rank; each rank checks the column
        blocks of its own tables against the CPU oracle (so every peer store path is covered)."""
        import torch

        from oracle import eb_oracle as O
        self.step(0)
        if self.bag is not None:
            self.bag.sync_result()
        torch.cuda.synchronize()
        per = -(-C4["bags"] // self.world)
        local_rows = np.arange(0, per, max(1, per // 256))
        sample = self._last[torch.from_numpy(local_rows).to(self.dev)].contiguous()
        if self.world > 1:
            import torch.distributed as dist
            parts = [torch.empty_like(sample) for _ in range(self.world)]
            dist.all_gather(parts, sample)
        else:
            parts = [sample]
        ok = True
        for r, part in enumerate(parts):
            got = part.cpu().numpy()
            take = local_rows + r * per
            keep = take < C4["bags"]
            take = take[keep]
            for t in self.here:
                if t in self.replicated and r != self.rank:
                    continue      # a replicated table's column is checked by the rank that pooled it
                b = self.bags[t]
                idx = b.indices.reshape(-1, self.L)[take].reshape(-1)
                w = b.per_sample_weights.reshape(-1, self.L)[take].reshape(-1)
                uniq, inv = np.unique(idx, return_inverse=True)
                compact = O.table_rows(uniq, self.dim, seed=300 + t, scale=0.1, dtype=np.float32)
                exp = O.pool(compact, inv.astype(np.int32), None, mode=O.MODE_SUM, fixed_len=self.L,
                             per_sample_weights=w, out_dtype=np.float32)
                ok = ok and bool(np.allclose(got[keep][:, t, :], exp, rtol=1e-5, atol=1e-6))
        if self.world > 1:
            flag = torch.tensor([1 if ok else 0], device=self.dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
        return ok

    def run_e2e(self, args):
        """Every step: one host-to-device copy per local table (indices + weights from pinned
        memory), the step, and this rank's result copied back to pinned memory.  N = 1: results
        alternate between two device buffers and go back on a second stream, so a step's
        copy-out overlaps the next step's copy-in and pooling."""
        import torch
        capi = self.capi
        self.step(0)
        if self.bag is not None:
            self.bag.sync_result()
        torch.cuda.synchronize()
        res = self.result()
        h_out = [torch.empty(tuple(res.shape), dtype=res.dtype).pin_memory() for _ in range(2)]
        steps = max(3, min(args.steps, 50))
        main = torch.cuda.current_stream()
        if self.world == 1:
            outs = [res, torch.empty_like(res)]
            params = [[capi.make_params(self.tables[t], self.d_idx[t], None, out=o[:, t, :],
                                        mode=self.mode, fixed_len=self.L,
                                        per_sample_weights=self.d_w[t]) for t in self.mine]
                      for o in outs]
            back = torch.cuda.Stream()
            pooled = [torch.cuda.Event() for _ in range(2)]
            copied = [torch.cuda.Event() for _ in range(2)]

            def step(k):
                j = k % 2
                for t in self.mine:
                    self.d_in[t].copy_(self.h_in[t], non_blocking=True)
                main.wait_event(copied[j])          # outs[j] was last read by the copy-out of step k-2
                for p in params[j]:
                    capi.forward(p, main.cuda_stream)
                pooled[j].record(main)
                with torch.cuda.stream(back):
                    back.wait_event(pooled[j])
                    h_out[j].copy_(outs[j], non_blocking=True)
                    copied[j].record(back)
        else:
            def step(k):
                for dst, src in self.copies:
                    dst.copy_(src, non_blocking=True)
                self.step(k)
                self.bag.sync_result()
                h_out[k % 2].copy_(self.result(), non_blocking=True)

        for k in range(3):
            step(k)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for k in range(steps):
            step(k)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if self.world > 1:
            tt = torch.tensor([dt], dtype=torch.float64, device=self.dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
        h2d = sum(src.numel() * 4 for _, src in self.copies)
        d2h = h_out[0].numel() * h_out[0].element_size()
        return {"value": self.T * C4["bags"] * self.L * steps / dt, "unit": "lookups/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": dt / steps * 1e3, "steps": steps, "note": "bytes are per rank",
                "api": "fwd_eb_forward per table" if self.world == 1 else "forward_b200.dist TableWiseBags.forward"}


def total_lookups(wl, steps: int, dev) -> float:
    """Whole-job lookups over `steps` steps: table-wise ranks each look up their own table."""
    n = float(sum(wl.lookups(k) for k in range(steps)))
    if wl.world > 1 and wl.workload in ("tablewise", "c4"):
        import torch
        import torch.distributed as dist
        t = torch.tensor([n], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        n = float(t.item())
    return n


REGIONS = 25            # timed regions of --steps steps each; `value` is the median region


def timed_regions(wl, steps: int, regions: int, barrier, multi: bool):
    """`regions` timed regions of exactly `steps` steps each.  Every region is bracketed by a
    barrier + synchronize on both sides and the start event is recorded directly after the
    barrier returns (nothing host-side in between, so ranks enter the region together).
    Returns the per-region milliseconds of THIS rank."""
    import torch
    begin = [torch.cuda.Event(enable_timing=True) for _ in range(regions)]
    end = [torch.cuda.Event(enable_timing=True) for _ in range(regions)]
    step = wl.step
    sync_result = wl.bag.sync_result if multi else None
    fork, join = getattr(wl, "fork", None), getattr(wl, "join", None)
    order = wl.bag.order_behind_current if multi else None
    for r in range(regions):
        barrier()
        begin[r].record()
        if order:
            order()          # N > 1: the step streams start behind the start event
        if fork:
            fork()           # N = 1: the other lanes' streams start behind the start event
        for k in range(steps):
            step(k)
        if sync_result:
            sync_result()    # the last step's fold / flag wait (side stream) is inside the region
        if join:
            join()           # ... and the end event waits for every lane
        end[r].record()
    barrier()
    return np.array([begin[r].elapsed_time(end[r]) for r in range(regions)])


def isolated_launch_us(wl, samples: int = 40):
    """One step at a time between its own pair of events, outside the timed regions: the pooling
    launch(es) of a step alone.  A few microseconds above the back-to-back figure (the events'
    own cost, and an event between two grids keeps the second from overlapping the first one's
    drain)."""
    import torch
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(samples)]
    for k in range(samples):
        wl.step(k, events=ev[k])
        ev[k][1].synchronize()     # one step at a time: with steps alternating over streams two would overlap
    if wl.bag is not None:
        wl.bag.sync_result()
    torch.cuda.synchronize()
    return np.array([a.elapsed_time(b) for a, b in ev]) * 1e3


def measure(workload: str, args, world: int, rank: int, dev, sampler=None, *, steps: int,
            regions: int, want_e2e: bool, want_cpu: bool, want_ref_kernel: bool, preheat_ms: float):
    """Build `workload` on this rank, time it, verify it, and return the pieces of a bench line
    (every rank computes them; rank 0 prints)."""
    import torch

    from forward_b200 import capi
    multi = world > 1
    dist = None
    if multi:
        import torch.distributed as dist
    wl = C4Workload(world, rank, dev, args) if workload == "c4" else \
        GpuWorkload(workload, world, rank, dev, args)

    def barrier():
        if multi:
            dist.barrier()
        torch.cuda.synchronize()

    # bring clocks up before the counted warm-up; a fixed count when ranks must stay in step
    if multi:
        for k in range(100 if workload == "c4" else int(preheat_ms * 4)):
            wl.step(k)
            if k % 64 == 63:
                torch.cuda.synchronize()
    else:
        t_end = time.perf_counter() + preheat_ms * 1e-3
        k = 0
        while time.perf_counter() < t_end:
            wl.step(k)
            k += 1
            if k % 64 == 0:
                torch.cuda.synchronize()
    pool_only_us = None
    if wl.pool_only:
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if hasattr(wl, "pool_fork"):
            wl.pool_fork()
        for k in range(20):
            wl.pool_only(k)
        if hasattr(wl, "pool_join"):
            wl.pool_join()
        n_po = max(20, min(steps, 200))
        a.record()
        if hasattr(wl, "pool_fork"):
            wl.pool_fork()
        for k in range(n_po):
            wl.pool_only(k)
        if hasattr(wl, "pool_join"):
            wl.pool_join()
        b.record()
        torch.cuda.synchronize()
        pool_only_us = a.elapsed_time(b) * 1e3 / n_po
    for k in range(args.warmup):
        wl.step(k)
    launches0 = capi.lib().fwd_eb_launch_count()
    if sampler:
        sampler.start()
    region_ms = timed_regions(wl, steps, regions, barrier, multi)
    clocks = sampler.stop() if sampler else None
    launches = (capi.lib().fwd_eb_launch_count() - launches0) // regions
    iso_us = isolated_launch_us(wl)
    host_us = None
    if multi:
        # what the host spends queueing one step (no synchronisation inside the loop): a step
        # cannot run faster than this
        barrier()
        # few enough steps that the launch queue never fills (a full queue would make the host wait
        # for the device and the figure would be device time)
        reps = max(5, min(100, 300 // max(1, getattr(wl, "launches_per_step", 1) + 3)))
        t0 = time.perf_counter()
        for k in range(reps):
            wl.step(k)
        host_us = (time.perf_counter() - t0) * 1e6 / reps
        wl.bag.sync_result()
        torch.cuda.synchronize()
    lookups = total_lookups(wl, steps, dev)
    exchange = None
    if multi:
        if wl.bag.check_status() != 0:
            raise RuntimeError("a bounded flag wait gave up during the timed regions")
        tt = torch.tensor(list(region_ms) + [pool_only_us], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)      # every region: the slowest rank's time
        region_ms, pool_only_us = tt[:-1].cpu().numpy(), float(tt[-1].item())
    total_ms = float(np.median(region_ms))
    if multi:
        step_us = total_ms * 1e3 / steps
        bags_n = wl.batches[0].num_bags
        egress = wl.egress_bytes() if hasattr(wl, "egress_bytes") else \
            bags_n * (world - 1) // world * wl.dim * wl.out_itemsize
        extra_us = max(step_us - pool_only_us, 1e-3)
        exchange = {"method": args.exchange + ("+ship" if args.ship and args.exchange in ("push", "compact") else ""),
                    "wire": "f16" if wl.out_itemsize == 2 else "f32",
                    "pool_only_us": pool_only_us, "step_us": step_us,
                    "overhead_frac": (step_us - pool_only_us) / pool_only_us,
                    "nvlink_egress_bytes_per_rank": int(egress),
                    "nvlink_floor_us_at_770GBs": egress / 770e9 * 1e6,
                    # this rank's egress over the whole step, against 900 GB/s per direction (the
                    # exchange runs beside the pooling: there is no exchange-only time to divide by)
                    "nvlink_frac": egress / (step_us * 1e-6) / 900e9,
                    # ... and over only the time a step takes longer than the pooling alone
                    "nvlink_frac_of_added_time": egress / (extra_us * 1e-6) / 900e9,
                    "host_us_per_step_queued": host_us}
    value = lookups / (total_ms * 1e-3)

    peak, peak_kind = measured_peak()
    if multi:
        # the pooling kernel(s) of a step with their peer stores, from the isolated launches
        alg = float(np.mean([wl.algorithmic_bytes(k) for k in range(len(iso_us))]))
        launch_ms = float(np.median(iso_us)) * 1e-3
        timed_by = "events around single steps, median of %d (outside the timed regions)" % len(iso_us)
    else:
        # a timed region holds nothing but the K pooling steps: average duration over the region
        alg = float(np.mean([wl.algorithmic_bytes(k) for k in range(steps)]))
        launch_ms = total_ms / steps
        timed_by = "events around the median timed region / steps"
    one_stream_us = None
    n_lanes = len(getattr(wl, "lane_streams", [])) if not multi else 0
    if n_lanes > 1:
        # the same steps back to back on ONE stream, for comparison (no overlap of consecutive grids)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        for k in range(steps):
            wl.step(k, lane=0)
        ev1.record()
        torch.cuda.synchronize()
        one_stream_us = ev0.elapsed_time(ev1) * 1e3 / steps
        timed_by += (f"; consecutive steps rotate over {n_lanes} streams, so this is the time per launch with "
                     "neighbouring grids overlapping (`kernel_us_one_stream`: the same steps on one stream)")
    achieved = alg / (launch_ms * 1e-3) / 1e9
    traffic, traffic_src = ncu_traffic(workload)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src,
                "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0,
                "kernel_us_mean": launch_ms * 1e3, "timed_by": timed_by,
                "kernel_us_isolated_median": float(np.median(iso_us)),
                "kernel_us_isolated_samples": int(len(iso_us)),
                "algorithmic_bytes_per_launch": alg}
    if traffic:
        # DRAM bytes per launch (ncu) over the same duration: what the memory system moved, beside
        # the algorithmic figure that counts every repeated row again
        roofline["dram_achieved"] = traffic / (launch_ms * 1e-3) / 1e9
        roofline["dram_frac"] = roofline["dram_achieved"] / peak
    if one_stream_us is not None:
        roofline["kernel_us_one_stream"] = one_stream_us
        roofline["streams"] = n_lanes
    if workload in ("c2", "tablewise"):
        roofline["note"] = ("Zipf indices: hot rows are served from L1 / L2 (DRAM traffic is `traffic`, a fifth of the "
                            "algorithmic bytes), so `frac` can exceed 1; the HBM-bound figure of this kernel is "
                            "`roofline_uniform` (same shape, uniform indices)")
    if workload == "c2u":
        roofline["note"] = ("uniform indices over a 256 MB table: the 126 MB L2 still serves about a fifth of the row "
                            "reads (`traffic` against `algorithmic_bytes_per_launch`), so `frac`, which counts every "
                            "repeated row, can exceed 1; `dram_frac` is what DRAM moved over the same time")
    if workload == "c4":
        roofline["launches_per_step"] = wl.launches_per_step
        roofline["note"] = "kernel_us_* and the bytes cover one step = all of this rank's tables"
        verified = None if args.no_verify else wl.verify()
        e2e = wl.run_e2e(args) if want_e2e else None
    else:
        verified = None if args.no_verify else verify(wl, workload, world, rank)
        e2e = None
        if want_e2e:
            e2e = run_e2e_multi(args, wl, rank, world, dev) if multi else run_e2e(args, wl)
            if not multi and not args.no_plugin_e2e:
                e2e["through_plugin_enqueue"] = run_e2e_plugin(args, wl)
    cpu = cpu_baseline(workload, world, args.cpu_seconds) if (want_cpu and rank == 0) else None
    ref_kernel = reference_kernel_side_by_side(wl) if want_ref_kernel else None
    out = {"value": value, "ms_per_step": total_ms / steps, "steps": steps, "regions": int(regions),
           "region_ms_min": float(region_ms.min()), "region_ms_median": total_ms,
           "region_ms_max": float(region_ms.max()),
           "roofline": roofline, "exchange": exchange, "verified": verified, "e2e": e2e,
           "cpu_baseline": cpu, "reference_kernel": ref_kernel, "gpu_launches": int(launches),
           "clocks": clocks, "config": describe(workload, world, args)}
    if multi:
        wl.bag.close()
    del wl
    torch.cuda.empty_cache()
    return out


def extra_object(m: dict) -> dict:
    """The short form of a secondary workload attached to the main line."""
    o = {"workload": m["config"]["workload"], "lookups_per_sec": m["value"],
         "us_per_step": m["ms_per_step"] * 1e3, "steps": m["steps"], "regions": m["regions"],
         "region_ms_min": m["region_ms_min"], "region_ms_max": m["region_ms_max"],
         "verified": m["verified"], "gpu_launches": m["gpu_launches"],
         "roofline": {k: m["roofline"][k] for k in ("achieved", "peak", "frac", "frac_of_8000", "traffic",
                                                     "kernel_us_mean", "algorithmic_bytes_per_launch",
                                                     "peak_kind")}}
    for k in ("kernel_us_one_stream", "streams", "dram_achieved", "dram_frac", "note"):
        if k in m["roofline"]:
            o["roofline"][k] = m["roofline"][k]
    if m["exchange"]:
        x = m["exchange"]
        o.update(step_us=x["step_us"], pool_only_us=x["pool_only_us"], overhead_frac=x["overhead_frac"],
                 nvlink_egress_bytes_per_rank=x["nvlink_egress_bytes_per_rank"],
                 nvlink_frac=x["nvlink_frac"], exchange=x["method"], wire=x["wire"])
    return o


def run_ours(args, world: int, rank: int, local_rank: int):
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the package has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    multi = world > 1
    if multi:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    # NVML is initialised here, long before any timed region; several ranks share the host's
    # cores, so they poll less often
    sampler = ClockSampler(local_rank, 0.001 if not multi else 0.004)
    workload = resolve_workload(args.workload, world)
    primary_steps = min(args.steps, 40) if workload == "c4" else args.steps
    main = measure(workload, args, world, rank, dev, sampler, steps=primary_steps, regions=args.regions,
                   want_e2e=not args.no_e2e, want_cpu=not multi and not args.no_cpu_baseline,
                   want_ref_kernel=(workload == "c2" and not multi), preheat_ms=args.preheat_ms)
    extras = {}
    if args.workload == "auto" and not args.no_extras:
        # the other configurations the metric is quoted on, in the same run: at N = 1 the
        # HBM-bound variants of the single-GPU path, at N > 1 the two multi-GPU configurations
        plan = [("roofline_uniform", "c2u", {}), ("c3", "c3", {})] if not multi else \
            [("c5", "c5", {"exchange": "compact", "wire": "f16"}), ("c4", "c4", {"exchange": "push"})]
        for key, name, over in plan:
            sub = argparse.Namespace(**vars(args))
            for k2, v2 in over.items():
                setattr(sub, k2, v2)
            try:
                m = measure(name, sub, world, rank, dev, None,
                            steps=min(args.steps, 20) if name == "c4" else min(args.steps, 400),
                            regions=7 if name == "c4" else min(args.regions, 15), want_e2e=False,
                            want_cpu=False, want_ref_kernel=False, preheat_ms=100.0)
                extras[key] = extra_object(m)
            except Exception as exc:    # a secondary workload must never cost the headline line
                extras[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                torch.cuda.synchronize()
    if rank == 0:
        line = {
            "metric": "pooled_lookups_per_sec", "value": main["value"], "unit": "lookups/s",
            "n_gpus": world, "steps": main["steps"], "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": scaling_kind(workload), "vs_baseline": None,
            "dtype": compute_dtype(workload), "table_dtype": "f32" if workload == "c4" else "f16",
            "data": "synthetic (table values: counter-based generator, Irwin-Hall bell of the "
                    "configuration's sigma; lengths and indices: the configuration's laws)",
            "config": main["config"], "regions": main["regions"],
            "region_ms_min": main["region_ms_min"], "region_ms_median": main["region_ms_median"],
            "region_ms_max": main["region_ms_max"],
            "roofline": main["roofline"], "cpu_baseline": main["cpu_baseline"], "e2e": main["e2e"],
            "gpu_launches": main["gpu_launches"], "clocks": main["clocks"],
            "verified_against_oracle": main["verified"],
        }
        if main["exchange"]:
            line["exchange"] = main["exchange"]
        if main["reference_kernel"]:
            line["reference_kernel"] = main["reference_kernel"]
        line.update(extras)
        print(json.dumps(line), flush=True)
    if multi:
        import torch.distributed as dist
        dist.destroy_process_group()


def reference_kernel_side_by_side(wl):
    """The reference's own EmbeddingBagCuda, recompiled unmodified for sm_100a, on the c2 batches
    with an fp32 copy of the table in sum mode (the only dtype it supports; its op codes for mean
    and max are wrong), next to our kernel on exactly those inputs.  None where the reference
    kernels were not built (the reference tree is not present on every machine)."""
    import torch

    from oracle import ref_kernels as R
    if not R.available():
        return None
    capi = wl.capi
    t32 = wl.table.float()
    bags_n = wl.batches[0].num_bags
    out_ref = torch.empty((bags_n, wl.dim), dtype=torch.float32, device=wl.dev)
    out_ours = torch.empty_like(out_ref)
    stream = torch.cuda.current_stream().cuda_stream
    params = [capi.make_params(t32, i, o, out=out_ours, mode=capi.MODE_SUM) for i, o in wl.d_batches]

    def timed(fn, n):
        for k in range(5):
            fn(k)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for k in range(n):
            fn(k)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / n

    for i_, o_ in wl.d_batches:     # checked once (the check synchronises), timed unchecked
        R.bag(i_, o_, out_ref, t32, 0, 0, stream)
    ref_us = timed(lambda k: R.bag(wl.d_batches[k % wl.nb][0], wl.d_batches[k % wl.nb][1], out_ref,
                                   t32, 0, 0, stream, check=False), 50)
    ours_us = timed(lambda k: capi.forward(params[k % wl.nb], stream), 200)
    R.bag(wl.d_batches[0][0], wl.d_batches[0][1], out_ref, t32, 0, 0, stream)
    capi.forward(params[0], stream)
    torch.cuda.synchronize()
    agree = bool(torch.allclose(out_ref, out_ours, rtol=1e-4, atol=1e-4))
    n = float(np.mean([b.num_indices for b in wl.batches]))
    return {"what": "reference EmbeddingBagCuda (embedding_bag_plugin.cu:66-118) recompiled for sm_100a, "
                    "c2 batches, fp32 table, sum",
            "reference_us": ref_us, "ours_same_inputs_us": ours_us, "speedup": ref_us / ours_us,
            "reference_lookups_per_sec": n / (ref_us * 1e-6), "outputs_agree": agree}


def verify(wl, workload, world, rank):
    """One more step after the timed regions, checked on every rank against the CPU oracle on a
    sample of the bags that rank ends up with (all ranks must agree for `true`).  The check is
    bit for bit wherever the order of the additions is defined: single-GPU and table-wise results
    (rows added in bag order), row shards (each window's partial in bag order, rounded to the wire
    type, the partials added in rank order).  Only NCCL's reduce-scatter, whose order is the
    library's, is compared within 1e-5."""
    import torch

    from oracle import eb_oracle as O
    wl.step(0)
    if wl.bag is not None:
        wl.bag.sync_result()
    torch.cuda.synchronize()
    res = wl.result()
    got = res.cpu().numpy()
    b = wl.batches[0]
    bags_n = b.num_bags
    per = -(-bags_n // world)
    lo = rank * per if world > 1 else 0
    stride = max(1, per // 512)
    take = np.arange(lo, min(lo + per, bags_n))[::stride]
    ends = np.append(b.offsets, b.num_indices).astype(np.int64)
    idx = np.concatenate([b.indices[ends[t]:ends[t + 1]] for t in take]).astype(np.int64)
    lens = np.array([ends[t + 1] - ends[t] for t in take])
    offs = np.zeros(take.size, dtype=np.int32)
    offs[1:] = np.cumsum(lens[:-1])
    uniq, inv = np.unique(idx, return_inverse=True)
    inv = inv.astype(np.int32)
    seed, scale = table_seed(workload, rank)
    compact = O.table_rows(uniq, wl.dim, seed=seed, scale=scale, dtype=np.float16)
    pad = -1
    if wl.pad >= 0:
        hit = int(np.searchsorted(uniq, wl.pad))
        pad = hit if hit < uniq.size and uniq[hit] == wl.pad else -1
    mode = {wl.capi.MODE_MEAN: O.MODE_MEAN, wl.capi.MODE_SUM: O.MODE_SUM,
            wl.capi.MODE_MAX: O.MODE_MAX}[wl.mode]

    def window(flo, fhi, m):
        """Partial of the logical row window [flo, fhi): `uniq` is sorted, so the window is a
        slice of the compact table and the oracle's own row filter does the rest."""
        a_, b_ = int(np.searchsorted(uniq, flo)), int(np.searchsorted(uniq, fhi))
        return O.pool(compact[a_:b_], inv, offs, mode=m, padding_idx=pad, row_lo=a_, out_dtype=np.float32)

    exact = True
    if workload == "tablewise":
        mine = got[take - lo, rank, :]        # column block of this rank's own table
        exp = O.pool(compact, inv, offs, mode=mode, padding_idx=pad)
    elif world == 1:
        mine = got[take - lo]
        if getattr(wl, "local_filter", None):   # one GPU holding one row window: that window's partial
            exp = window(*wl.local_filter, mode).astype(np.float16)
        else:
            exp = O.pool(compact, inv, offs, mode=mode, padding_idx=pad)
    else:
        mine = got[take - lo]
        ex = wl.args.exchange
        sums_then_divide = ex == "compact" and mode == O.MODE_MEAN
        total_rows = C5["rows"] if workload == "c5" else C2["rows"] * world
        parts = []
        for r in range(world):
            if workload == "c5":
                flo, n_r = wl.fd.shard_rows(total_rows, world, r)
            else:
                flo, n_r = r * C2["rows"], C2["rows"]
            parts.append(window(flo, flo + n_r, O.MODE_SUM if sums_then_divide else mode))
        parts = np.stack(parts)
        if wl.out_itemsize == 2:
            parts = parts.astype(np.float16)
        exp = O.combine_partials(parts, np.float32)
        if sums_then_divide:
            exp = (exp / np.maximum(lens, 1)[:, None].astype(np.float32)).astype(np.float32)
        exact = ex != "nccl"
    if exact:
        mine, exp = np.ascontiguousarray(mine), np.ascontiguousarray(exp)
        if mine.dtype != exp.dtype:     # a variant that returns another type: compare values
            ok = bool(np.allclose(mine.astype(np.float32), exp.astype(np.float32), rtol=1e-3, atol=1e-3))
        else:
            bits = np.uint16 if mine.dtype == np.float16 else np.uint32
            ok = bool(np.array_equal(mine.view(bits), exp.view(bits)))
    else:
        ok = bool(np.allclose(mine, exp, rtol=1e-5, atol=1e-5))
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([1 if ok else 0], device=wl.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = bool(t.item())
    return ok


_HOST_TABLES = {}


def run_e2e_plugin(args, wl):
    """N = 1, the same steps through the EmbeddingBag_TRT plugin object instead of the session:
    the plugin is built from a host copy of the table (description -> layer creator -> createPlugin
    -> clone -> configurePlugin, as TensorRT would), and every step copies one batch's indices and
    offsets from pinned host memory, calls the plugin's enqueue on a stream of its own and copies
    the pooled rows back; four steps in flight.  The plugin's tensors have fixed shapes, so every
    step reuses batch 0."""
    import ctypes as C

    import torch
    capi = wl.capi
    lib_path = os.path.join(ROOT, "forward_b200", "lib", "libfwd_eb_plugin.so")
    if not os.path.exists(lib_path):
        return {"unavailable": "libfwd_eb_plugin.so is not built"}
    h = C.CDLL(lib_path)
    h.fwd_eb_host_build.restype = C.c_void_p
    h.fwd_eb_host_build.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                    C.c_void_p, C.c_int, C.c_void_p]
    h.fwd_eb_host_free.argtypes = [C.c_void_p]
    h.fwd_eb_host_run.argtypes = [C.c_void_p] * 6
    b = wl.batches[0]
    seed, scale = table_seed(wl.workload, 0)
    key = (wl.workload, seed)
    if key not in _HOST_TABLES:
        _HOST_TABLES[key] = host_table(wl.table.shape[0], wl.dim, wl.row_lo, seed, scale)
    table = _HOST_TABLES[key]
    idx_dims = (C.c_int * 1)(b.num_indices)
    off_dims = (C.c_int * 1)(b.num_bags)
    plugin = h.fwd_eb_host_build(table.ctypes.data, 1, table.shape[0], table.shape[1], 0, int(wl.mode),
                                 int(wl.pad), 0, 1, 1, idx_dims, 1, off_dims, 0, None)
    if not plugin:
        return {"unavailable": "the plugin refused the configuration"}
    depth = 4
    dev = wl.dev
    h_in = [torch.cat([torch.from_numpy(b.offsets), torch.from_numpy(b.indices)]).pin_memory()
            for _ in range(depth)]
    d_in = [torch.empty_like(x, device=dev) for x in h_in]
    d_out = [torch.empty((b.num_bags, wl.dim), dtype=torch.float16, device=dev) for _ in range(depth)]
    h_out = [torch.empty((b.num_bags, wl.dim), dtype=torch.float16).pin_memory() for _ in range(depth)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(depth)]
    done = [torch.cuda.Event() for _ in range(depth)]
    nb = b.num_bags

    def step(k):
        j = k % depth
        done[j].synchronize()                    # result of the step issued `depth` steps ago
        _ = float(h_out[j][0, 0])                # touch it
        with torch.cuda.stream(streams[j]):
            d_in[j].copy_(h_in[j], non_blocking=True)
            rc = h.fwd_eb_host_run(plugin, d_in[j][nb:].data_ptr(), d_in[j][:nb].data_ptr(), None,
                                   d_out[j].data_ptr(), streams[j].cuda_stream)
            if rc != 0:
                raise RuntimeError(f"plugin enqueue returned {rc}")
            h_out[j].copy_(d_out[j], non_blocking=True)
            done[j].record(streams[j])

    torch.cuda.synchronize()
    for k in range(max(args.warmup, depth)):
        step(k)
    torch.cuda.synchronize()
    steps = args.steps
    t0 = time.perf_counter()
    for k in range(steps):
        step(k)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    # the plugin's result on batch 0 must be the C-ABI path's, bit for bit
    wl.step(0)
    torch.cuda.synchronize()
    same = bool(torch.equal(wl.result().view(torch.int16), d_out[(steps - 1) % depth].view(torch.int16)))
    h.fwd_eb_host_free(plugin)
    return {"value": b.num_indices * steps / dt, "unit": "lookups/s", "ms_per_step": dt / steps * 1e3,
            "h2d_bytes_per_step": int(h_in[0].numel() * 4), "d2h_bytes_per_step": int(h_out[0].numel() * 2),
            "calls_in_flight": depth, "equals_c_abi_result": same,
            "api": "EmbeddingBagPlugin::enqueue (TensorRT call order; interface stand-in)"}


def run_e2e(args, wl):
    """N = 1: the same calls through the host-buffer session: pinned inputs in, result out, each
    step, `depth` calls in flight."""
    import torch

    from forward_b200.session import Session
    capi = wl.capi
    depth = args.e2e_depth
    max_n = max(b.num_indices for b in wl.batches)
    bags_n = wl.batches[0].num_bags
    s = Session(table_dtype=capi.F16, dim=wl.dim, num_rows=wl.table.shape[0], mode=wl.mode,
                max_indices=max_n, max_bags=bags_n, depth=depth, external_table=True,
                padding_idx=wl.pad, row_lo=wl.row_lo)
    s.adopt_table(wl.table.data_ptr())
    views = [s.slot(k) for k in range(depth)]
    sizes = []
    for k in range(depth):       # slot k carries batch k; its copy-in still happens every step
        b = wl.batches[k % wl.nb]
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


def run_e2e_multi(args, wl, rank, world, dev):
    """N > 1: every step copies this rank's batch from pinned host memory to its GPU, runs the
    multi-GPU call and copies this rank's slice of the result back to pinned memory."""
    import torch
    import torch.distributed as dist
    # offsets and indices of a batch share one pinned block and go up as ONE copy (a second,
    # small copy per step costs far more copy-engine time than its bytes)
    host = [torch.cat([torch.from_numpy(b.offsets), torch.from_numpy(b.indices)]).pin_memory()
            for b in wl.batches]
    d_in = [torch.empty_like(h, device=dev) for h in host]
    d_off = [d[:b.offsets.size] for d, b in zip(d_in, wl.batches)]
    d_idx = [d[b.offsets.size:] for d, b in zip(d_in, wl.batches)]
    wl.step(0)
    wl.bag.sync_result()
    torch.cuda.synchronize()
    shape, dtype = tuple(wl.result().shape), wl.result().dtype
    h_out = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(wl.nb)]
    saved = wl.d_batches
    wl.set_device_batches(list(zip(d_idx, d_off)))
    wl.resident = False      # every step's inputs now arrive by a copy on the current stream

    def step(k):
        j = k % wl.nb
        d_in[j].copy_(host[j], non_blocking=True)
        wl.step(k)
        side = wl.bag.side                      # with "push" the result completes on a side stream
        if side is not None:
            with torch.cuda.stream(side):
                h_out[j].copy_(wl.result(), non_blocking=True)
        else:
            h_out[j].copy_(wl.result(), non_blocking=True)

    for k in range(max(args.warmup, 3)):
        step(k)
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for k in range(args.steps):
        step(k)
    torch.cuda.synchronize()
    stats = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    dt = float(stats.item())
    wl.set_device_batches(saved)
    lookups = total_lookups(wl, args.steps, dev)
    h2d = int(np.mean([b.num_indices * 4 + b.num_bags * 4 for b in wl.batches]))
    d2h = int(np.prod(shape)) * h_out[0].element_size()
    return {"value": lookups / dt, "unit": "lookups/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": dt / args.steps * 1e3,
            "note": "bytes are per rank; at N > 1 this leg is bound by the host (N processes share its memory "
                    "bandwidth and cores for the pinned copies), not by the GPUs or NVLink",
            "api": "forward_b200.dist forward()"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto",
                    choices=["auto", "c2", "c2u", "tablewise", "rowshard", "c5", "c3", "c4"])
    ap.add_argument("--streams", type=int, default=2,
                    help="N=1: consecutive steps (independent batches) rotate over this many streams, each "
                         "with its own output buffer; 1 = every step on one stream")
    ap.add_argument("--regions", type=int, default=REGIONS,
                    help="timed regions of --steps steps each (barrier before each); `value` is the "
                         "median region")
    ap.add_argument("--no-extras", action="store_true",
                    help="--workload auto: skip the secondary workloads attached to the line "
                         "(N=1: uniform-index c2 and c3; N>1: c5 and c4)")
    ap.add_argument("--no-plugin-e2e", action="store_true")
    ap.add_argument("--lookback", default=None,
                    help="N>1: EVERY,DEPTH of the exchange pipeline (fwd_eb_pipeline_set_lookback); "
                         "default: the library's 6,2")
    ap.add_argument("--ship", type=int, default=0, choices=[0, 1],
                    help="N>1, exchanges push / compact: 1 = the pooling kernel stores its rows locally and a "
                         "copy kernel on the side stream sends them to their owners; 0 = the pooling "
                         "kernel stores into the peers' buffers itself (the default: shipping measured "
                         "slower at 2 and at 8 GPUs)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "compact", "push", "stage", "a2a", "nccl"],
                    help="N>1: how pooled rows / partial bags reach their owners.  push: the pooling "
                         "kernel's own peer stores; compact (row shards only): window compaction first, "
                         "then push from the dense sub-bags; stage (row shards only): plain pooling, then "
                         "copy-engine transfers; a2a / nccl: NCCL collectives.  auto = compact for row "
                         "shards (the fastest there), push for table-wise placement")
    ap.add_argument("--wire", default="f32", choices=["f32", "f16"],
                    help="row shards with --exchange push: element type of the partials on NVLink")
    ap.add_argument("--c5-rows", type=int, default=C5["rows"],
                    help="c5: rows of the whole table (default 1e9; a smaller table for profiler captures)")
    ap.add_argument("--c5-window", type=int, default=1,
                    help="c5 at N=1: hold only one of this many row windows of the table and pool "
                         "that rank's partial bags (the per-rank kernel of a sharded run; no exchange)")
    ap.add_argument("--c4-replicate-mb", type=int, default=256,
                    help="c4 at N>1: tables smaller than this many MiB live on every rank, which pools its "
                         "own bags of them (no exchange); 0 = every table on one rank only")
    ap.add_argument("--local-streams", type=int, default=None, choices=[0, 1, 2],
                    help="c4: auxiliary streams for independent tables (N=1: 0 = one stream, else "
                         "fwd_eb_forward_many; N>1: streams for the replicated tables; default: the library's)")
    ap.add_argument("--c4-max-rows", type=int, default=0,
                    help="c4: cut every table to this many rows (0 = the configuration's sizes; a smaller "
                         "case for profiler captures)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-depth", type=int, default=4, help="N=1 e2e: calls in flight (1..16)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--preheat-ms", type=float, default=400.0,
                    help="untimed launches before the counted warm-up, to bring clocks up")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.lookback = tuple(int(v) for v in args.lookback.split(",")) if args.lookback else None
    C5["rows"] = args.c5_rows
    if args.exchange == "auto":
        args.exchange = "compact" if args.workload in ("rowshard", "c5") else "push"
    if args.exchange in ("stage", "compact") and args.workload not in ("rowshard", "c5"):
        raise SystemExit(f"--exchange {args.exchange} is for the row-sharded workloads (rowshard, c5)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run "
                         "(--nproc-per-node N)")
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    run_ours(args, world, rank, local_rank)


if __name__ == "__main__":
    main()
