#!/usr/bin/env python
"""Benchmark of the replay sample + gather hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one prioritized sample + gather of a batch: rebuild the cumulative
priority table (scan), draw B segment starts on supplied variates, gather B x L
timesteps of every column.

N = 1 runs the HBM-resident decision-transformer table (100,000 trajectories x
1000 steps, rows 156/24/4/4/1 B, B=1024, L=64) and, beside it under
`other_configs`, the index-only workload (1,048,576 priorities, 4096 variates),
the zero-copy workload (table in pinned mapped host memory, B=512, L=32) and the
sharded workload's whole global batch on this one GPU (the N = 1 point of ITS curve).
N > 1 runs the trajectory-id sharded token table (per GPU 32,000 x 1000 steps of
4104 B, global batch 8192, L=16) with the cross-shard exchange.

The line printed by rank 0 carries, beside the base keys:
  roofline      the dominant kernel (scan) against the measured HBM copy peak
  cpu_baseline  the CPU path timed on this box's host cores (bounded sample)
  e2e           the same metric through the C ABI with host buffers
  parity        indices/bytes of one batch checked against the CPU oracle
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "sampled timesteps/sec (prioritized sample + gather)"
UNIT = "timesteps/s"

C3 = dict(name="hbm_decision_transformer_100Mstep", rows=[156, 24, 4, 4, 1], T=1000, capacity=100_000,
          B=1024, L=64)
C5 = dict(name="sharded_token_table_32Mstep_per_gpu", rows=[4096, 4, 4], T=1000, capacity=32_000,
          B_global=8192, B_per_rank=1024, L=16)

# dram__bytes_read.sum + dram__bytes_write.sum of one scan_kernel launch at n = 100,000,000, taken
# once from a one-pass ncu capture of that launch (a profiler counter: it cannot be read inside a
# timed run; the part of the 400 MB of output that is still dirty in L2 at kernel end is not in it).
SCAN_TRAFFIC_BYTES_C3 = 741_204_736
# The same for the totals-only instance (no level-2 table written): 400,064,768 B read + 338,688 B written.
SCAN_TOTALS_TRAFFIC_BYTES_C3 = 400_403_456
TRAFFIC_SOURCE = "ncu capture of one launch at this size (dram__bytes_read.sum + dram__bytes_write.sum), not read in this run"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi samples of the SM clock and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            deadline = time.time() + 3.0      # nvidia-smi needs a few hundred ms before its first line
            while not self.rows and time.time() < deadline:
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        inside = [r for (t, r) in self.rows if t0 <= t <= t1 + 0.05] or [r for (_, r) in self.rows]
        sm, mx, reasons = [], [], set()
        for r in inside:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def fill_table(core, N, table, seed):
    """Seeded synthetic bytes for the whole table, written in HBM."""
    core.fill_ptr(table.device_ptr, table.nbytes // 4, N.FILL_U32, seed=seed)
    if table.nbytes % 4:
        core.fill_ptr(table.device_ptr + (table.nbytes // 4) * 4, table.nbytes % 4, N.FILL_U8, seed=seed + 1)


def run_ours_single(args):
    import numpy as np
    import torch
    from gear_b200 import _native as N
    from gear_b200 import core

    cfg = C3
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    core.init(0)
    rows, T, cap, B, L = cfg["rows"], cfg["T"], cfg["capacity"], cfg["B"], cfg["L"]
    n = cap * T
    cols = list(range(len(rows)))

    table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    table.connect()
    fill_table(core, N, table, seed=0x6EA20003)
    handler = core.StorageHandler(table)
    handler.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))

    prio = torch.empty(n, dtype=torch.float32, device=dev)
    core.fill(prio, N.FILL_F32_LOGNORMAL, seed=0x6EA20103)
    sampler = core.PrioritySampler(n)
    sampler_b = core.PrioritySampler(n)      # the stored-table mode alternates between two tables

    # variates: a fresh batch per step, all resident before the clock starts
    nbatches = 16
    u_dev = torch.empty(nbatches * B, dtype=torch.float64, device=dev)
    core.fill(u_dev, N.FILL_U01_F64, seed=0x6EA20203)
    dsts = [torch.empty(B * L * r, dtype=torch.uint8, device=dev) for r in rows]
    flat = torch.empty(B, dtype=torch.int64, device=dev)

    def batch(i):
        return u_dev[(i % nbatches) * B:(i % nbatches + 1) * B]

    K = args.steps
    clocks = ClockSampler(0)

    def timed_steps(store, sample_clocks):
        """K full steps (scan + one-launch search/decode/gather), timed as a whole with one pair of
        events; then an instrumented run of the same steps with an event after each of the step's three
        launches, from which only the kernels' own durations are taken (events between the
        launches cost the overlap of one kernel's start with its predecessor's end).
        store=True: the scan writes the level-2 table and the sampling kernel searches it;
        store=False: the scan keeps only the partition offsets and the sampling kernel rebuilds
        the one partition each request falls into from the priorities."""
        # The storing mode keeps TWO tables and uses them in turn, so that the scan of one may start
        # while the sampling launch that still reads the other finishes (the totals-only scan
        # overwrites nothing the sampling launch reads and needs no second table for that).
        tables = [sampler, sampler_b] if store else [sampler, sampler]

        def one_step(i):
            sm = tables[i & 1]
            sm.scan(prio, store=store, alternate=store)
            sm.sample_gather(handler, batch(i), cols, dsts, scale=True, zero_fill=True, out_flat=flat)

        # The clock sampler starts first and the GPU is brought to its working clocks by 60 ms of the
        # same steps (untimed, before the warm-up steps proper): a timed region of a few milliseconds
        # right after an idle GPU would otherwise be measured partly at idle clocks.
        if sample_clocks:
            clocks.start()
        t_load = time.time()
        spin_until = time.perf_counter() + 0.06
        i_spin = 0
        while time.perf_counter() < spin_until:
            one_step(i_spin)
            i_spin += 1
            if i_spin % 64 == 0:
                torch.cuda.synchronize()
        for i in range(max(args.warmup, 3)):
            one_step(i)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        t0 = time.time()
        ev[0].record()
        for i in range(K):
            one_step(i)
        ev[1].record()
        torch.cuda.synchronize()
        t1 = time.time()
        clk = clocks.stop(t_load, t1) if sample_clocks else None
        ms_step = ev[0].elapsed_time(ev[1]) / K
        Ki = min(K, 300)
        marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(Ki)]
        for i in range(Ki):
            marks[i][0].record()
            sampler.scan_partitions(prio, store=store)
            marks[i][1].record()
            sampler.scan_level1()
            marks[i][2].record()
            sampler.sample_gather(handler, batch(i), cols, dsts, scale=True, zero_fill=True, out_flat=flat)
            marks[i][3].record()
        torch.cuda.synchronize()
        scan_ev_ms = sum(m[0].elapsed_time(m[1]) for m in marks) / Ki
        level1_ms = sum(m[1].elapsed_time(m[2]) for m in marks) / Ki
        sample_ms = sum(m[2].elapsed_time(m[3]) for m in marks) / Ki
        # The scan kernel's own duration: launches of it alone, one behind the other with nothing in
        # between (strictly serialised: a scan of a sampler never starts beside the one before it), between
        # one pair of events.  An event on either side of a single launch adds about 5 us that are
        # not the kernel's (the ncu launch list agrees with this loop to 0.5 us).
        Kb = max(20, min(K, 200))
        for _ in range(3):
            sampler.scan_partitions(prio, store=store)
        torch.cuda.synchronize()
        eb = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        eb[0].record()
        for _ in range(Kb):
            sampler.scan_partitions(prio, store=store)
        eb[1].record()
        torch.cuda.synchronize()
        sampler.scan_level1()
        scan_ms = eb[0].elapsed_time(eb[1]) / Kb
        return ms_step, scan_ms, (level1_ms, sample_ms, scan_ev_ms), clk

    stored_ms, stored_scan_ms, stored_sample_ms, _ = timed_steps(True, False)
    ms_step, scan_ms, sample_ms, clk = timed_steps(False, True)          # the headline
    total_prio, status = sampler.result()

    gathered = B * L * sum(rows)
    value = B * L / (ms_step * 1e-3)
    peak, peak_src = peaks()
    nparts = (n + 4095) // 4096
    scan_bytes = 4 * n + 8 * nparts                    # totals-only scan: priorities read, offsets written
    stored_scan_bytes = 8 * n + 8 * nparts             # storing scan: also 4 B written per priority
    achieved = scan_bytes / (scan_ms * 1e-3) / 1e9
    stored_achieved = stored_scan_bytes / (stored_scan_ms * 1e-3) / 1e9
    step_bytes = scan_bytes + 2 * gathered + B * 4096 * 4   # + one 16 KiB partition re-read per request
    stored_step_bytes = stored_scan_bytes + 2 * gathered

    # ---- search + gather only ("priorities unchanged" mode), reported beside the headline
    e2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    sampler.scan(prio, store=False)
    e2[0].record()
    for i in range(K):
        sampler.sample_gather(handler, u_dev[(i % nbatches) * B:(i % nbatches + 1) * B], cols, dsts,
                              scale=True, zero_fill=True, out_flat=flat)
    e2[1].record()
    torch.cuda.synchronize()
    sg_ms = e2[0].elapsed_time(e2[1]) / K

    # ---- incremental mode: the B priorities of the previous batch change, only their partitions
    #      are rescanned (reported beside the headline; the headline rescans everything)
    new_val = torch.empty(nbatches * B, dtype=torch.float32, device=dev)
    core.fill(new_val, N.FILL_F32_LOGNORMAL, seed=0x6EA20303)
    e3 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    sampler.scan(prio, store=False)
    e3[0].record()
    for i in range(K):
        j = i % nbatches
        sampler.update(prio, flat, new_val[j * B:(j + 1) * B])     # the indices drawn by the previous step
        sampler.sample_gather(handler, u_dev[j * B:(j + 1) * B], cols, dsts, scale=True, zero_fill=True, out_flat=flat)
    e3[1].record()
    torch.cuda.synchronize()
    upd_ms = e3[0].elapsed_time(e3[1]) / K

    # ---- end to end through the public API with host buffers (pinned): variates in, batch out.
    #      Two batches in flight: the copy-out of a batch overlaps the sampling of the next
    #      (gear_b200.pipeline.HostBatchPipeline); `serial` is the same with one batch at a time.
    from gear_b200.pipeline import HostBatchPipeline
    u_host = torch.empty(nbatches * B, dtype=torch.float64).pin_memory()
    u_host.copy_(u_dev.cpu())
    Ke = max(10, min(K, 400))

    def e2e_run(depth):
        pipe = HostBatchPipeline(sampler, handler, cols, B, depth=depth)
        ub = lambda i: u_host[(i % nbatches) * B:(i % nbatches + 1) * B]
        for i in range(4):
            pipe.submit(prio, ub(i))
            if i >= depth - 1:
                pipe.next()
        pipe.drain()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for i in range(Ke):
            pipe.submit(prio, ub(i))
            if i >= depth - 1:
                pipe.next()                     # the caller holds a complete batch in host memory here
        pipe.drain()
        torch.cuda.synchronize()
        return (time.perf_counter() - w0) / Ke, pipe

    serial_s, _ = e2e_run(1)
    e2e_s, pipe = e2e_run(2)
    e2e = {"value": B * L / e2e_s, "unit": UNIT, "h2d_bytes_per_step": B * 8,
           "d2h_bytes_per_step": gathered + B * 8, "ms_per_step": e2e_s * 1e3, "steps": Ke,
           "batches_in_flight": 2,
           "serial": {"value": B * L / serial_s, "ms_per_step": serial_s * 1e3, "batches_in_flight": 1}}
    # the loader as the reference uses it: the batch stays in device memory for the trainer
    # (gear/loader/offline_loader.py:178-203 gathers into CUDA tensors); variates come from pinned
    # host memory and the drawn step ids go back to it; two batches in flight, and one at a time
    def device_batch_run(depth):
        p2 = HostBatchPipeline(sampler, handler, cols, B, depth=depth, batch_to_host=False)
        ub = lambda i: u_host[(i % nbatches) * B:(i % nbatches + 1) * B]
        for i in range(4):
            p2.submit(prio, ub(i))
            if i >= depth - 1:
                p2.next()
        p2.drain()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for i in range(Ke):
            p2.submit(prio, ub(i))
            if i >= depth - 1:
                p2.next()
        p2.drain()
        torch.cuda.synchronize()
        return (time.perf_counter() - w0) / Ke

    dev_serial_s, dev_batch_s = device_batch_run(1), device_batch_run(2)
    e2e["batch_left_in_hbm"] = {"value": B * L / dev_batch_s, "ms_per_step": dev_batch_s * 1e3, "batches_in_flight": 2,
                                "serial": {"value": B * L / dev_serial_s, "ms_per_step": dev_serial_s * 1e3},
                                "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8,
                                "note": "variates from pinned host memory, drawn ids back to it, the gathered batch "
                                        "stays in device memory as in the reference's loader"}
    # the last pipelined batch, in host memory, against the device-side result of the same variates
    hc, hf = pipe._host_cols[(Ke - 1) % 2], pipe._host_flat[(Ke - 1) % 2]
    sampler.scan(prio, store=False)
    sampler.sample_gather(handler, batch(Ke - 1), cols, dsts, scale=True, zero_fill=True, out_flat=flat)
    torch.cuda.synchronize()
    e2e["matches_device_result"] = bool(torch.equal(hf, flat.cpu()) and all(
        torch.equal(h, d.cpu()) for h, d in zip(hc, dsts)))

    # ---- parity of one batch against the CPU oracle + CPU baseline (bounded sample)
    core.fill(prio, N.FILL_F32_LOGNORMAL, seed=0x6EA20103)      # undo the incremental mode's updates
    parity, cpu = cpu_check_and_baseline(cfg, table, prio, u_dev[:B], sampler, handler, dsts, flat, args, store=False)
    parity_stored, _ = cpu_check_and_baseline(cfg, table, prio, u_dev[:B], sampler, handler, dsts, flat, args,
                                              store=True, want_cpu=False)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 scan / f64 level-1 / u8 gather", "data": "synthetic (seeded Philox4x32-10, generated in HBM)",
        "config": {"workload": cfg["name"], "trajectories": cap, "trajectory_length": T, "row_bytes": rows,
                   "batch": B, "segment_length": L, "priorities": n, "table_bytes": table.nbytes,
                   "l2": "inputs larger than L2 (400 MB of priorities re-read every step)",
                   "spin_up": "60 ms of untimed steps before the warm-up steps bring the GPU from idle to its working clocks; the clock samples (every 50 ms) cover that stretch and the timed region behind it",
                   "step": "totals-only scan (partition aggregates, block totals and superblock sums, no stored "
                           "level-2 table) + one launch that finds each request's partition through those sums, "
                           "rebuilds the one 512-value block it falls into, decodes and gathers; the level-1 "
                           "launch of a step runs beside the scan of the next (three launches per step, two on "
                           "the critical path)"},
        "gathered_gb_s": 2 * gathered / (ms_step * 1e-3) / 1e9,
        "step_algorithmic_gb_s": step_bytes / (ms_step * 1e-3) / 1e9,
        "step_frac_of_measured_peak": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
        "step_frac_of_8tbs": step_bytes / (ms_step * 1e-3) / 1e9 / 8000.0,
        "stored_table_mode": {
            "step": "scan that stores the level-2 table (8 B per priority) + level 1 + search + decode + gather; two "
                    "tables used in turn, so a scan may start while the sampling launch on the other table finishes",
            "ms_per_step": stored_ms, "timesteps_per_s": B * L / (stored_ms * 1e-3),
            "scan_ms": stored_scan_ms, "scan_ms_with_an_event_on_either_side": stored_sample_ms[2], "level1_ms": stored_sample_ms[0], "sample_gather_ms": stored_sample_ms[1], "scan_algorithmic_bytes": stored_scan_bytes,
            "scan_achieved_gb_s": stored_achieved, "scan_frac_of_measured_peak": stored_achieved / peak,
            "scan_traffic": SCAN_TRAFFIC_BYTES_C3,
            "step_algorithmic_gb_s": stored_step_bytes / (stored_ms * 1e-3) / 1e9,
            "step_frac_of_measured_peak": stored_step_bytes / (stored_ms * 1e-3) / 1e9 / peak,
            "step_frac_of_8tbs": stored_step_bytes / (stored_ms * 1e-3) / 1e9 / 8000.0, "parity": parity_stored},
        "search_gather_only": {"ms_per_step": sg_ms, "timesteps_per_s": B * L / (sg_ms * 1e-3),
                               "gathered_gb_s": 2 * gathered / (sg_ms * 1e-3) / 1e9},
        "incremental_update": {"ms_per_step": upd_ms, "timesteps_per_s": B * L / (upd_ms * 1e-3),
                               "step": f"update {B} priorities (rescan of the touched partitions + level 1) + "
                                       "search + decode + gather"},
        "roofline": {"kernel": "scan_kernel<false> (totals only)", "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "traffic": SCAN_TOTALS_TRAFFIC_BYTES_C3,
                     "traffic_source": TRAFFIC_SOURCE, "peak_source": peak_src, "algorithmic_bytes": scan_bytes, "avg_launch_ms": scan_ms,
                     "avg_launch_ms_how": "launches of the kernel alone, back to back and serialised, between one pair of events",
                     "avg_launch_ms_with_an_event_on_either_side": sample_ms[2],
                     "frac_with_an_event_on_either_side": scan_bytes / (sample_ms[2] * 1e-3) / 1e9 / peak,
                     "level1_cluster_kernel_ms": sample_ms[0], "sample_gather_kernel_ms": sample_ms[1],
                     "note": "the three launch times are taken with an event on either side of each launch, one "
                             "after the other; in the step the level-1 launch runs beside the next scan and the "
                             "sampling launch beside that scan's start, so ms_per_step is less than their sum"},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": 3 * K, "clocks": clk, "parity": parity,
        "scan_status": status, "total_priority": total_prio,
    }
    # ---- the other single-GPU configurations, on the same record
    del pipe, sampler, sampler_b, handler, table, prio, dsts, u_dev
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    other = {}
    def run_one_shard(a):
        # config 5 with its whole global batch on ONE GPU: the N = 1 point of the sharded
        # configuration's own scaling curve (the lines for N > 1 are that configuration)
        import bench_sharded
        a.steps, a.warmup = min(a.steps, 50), min(max(a.warmup, 3), 5)
        full = bench_sharded.run(a, emit=False)
        keep = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "config", "global_batch_8192",
                "global_batch_1024_per_gpu", "small_case_every_byte_vs_oracle", "roofline", "e2e", "parity", "gpu_launches")
        return {k: full[k] for k in keep if k in full}

    for name, fn in (("c2_index_sampling_only", run_index_only), ("c4_zero_copy_host_table", run_zero_copy),
                     ("c5_sharded_table_on_one_gpu", run_one_shard)):
        try:
            sub_args = argparse.Namespace(**vars(args))
            sub_args.steps = min(args.steps, 2000)
            other[name] = fn(sub_args)
        except Exception as e:  # reported, not fatal: the headline above stands on its own
            other[name] = {"error": f"{type(e).__name__}: {e}"}
        gc.collect()
        torch.cuda.empty_cache()
    line["other_configs"] = other
    print(json.dumps(line))


def cpu_check_and_baseline(cfg, table, prio, u_first, sampler, handler, dsts, flat, args, store=True, want_cpu=True):
    """One batch checked against the oracle, then the CPU path timed on a bounded sample."""
    import numpy as np
    import torch
    from oracle import oracle as O

    rows, T, cap, B, L = cfg["rows"], cfg["T"], cfg["capacity"], cfg["B"], cfg["L"]
    cols = list(range(len(rows)))
    cores = os.cpu_count() or 1
    hp = prio.cpu().numpy()
    u = u_first.cpu().numpy()

    # GPU result of exactly this batch
    sampler.scan(prio, store=store)
    sampler.sample_gather(handler, u_first.contiguous(), cols, dsts, scale=True, zero_fill=True, out_flat=flat)
    torch.cuda.synchronize()
    gflat = flat.cpu().numpy()

    t0 = time.perf_counter()
    ocdf, ol1, ototal, _ = O.scan_mt(hp, cores)
    scan_s = time.perf_counter() - t0
    oflat, near = O.search(ocdf, ol1, u, scale=True, want_near=True)
    oi, ot, ol = O.decode(oflat, T)
    index_mismatch = int((gflat != oflat).sum())
    f64 = O.search_f64(hp, u * ototal)
    flips = oflat != f64
    byte_mismatch = 0
    for c, r in enumerate(rows):
        s, d, b, slot = handler.sub(oi, ot, ol, c)
        got = dsts[c].cpu().numpy()
        for i in range(B):            # every request read back from the device table
            want = table.read(int(s[i]), int(b[i]))
            byte_mismatch += int((got[d[i]:d[i] + b[i]] != want).sum()) + int(got[i * slot + b[i]:(i + 1) * slot].any())
    parity = {"index_mismatches_vs_oracle": index_mismatch, "gathered_byte_mismatches": byte_mismatch,
              "requests_byte_checked": B, "variates_within_1ulp_of_boundary": int(near.sum()),
              "flips_vs_float64_running_sum": int(flips.sum()),
              "max_flip_distance": int(np.abs(oflat[flips] - f64[flips]).max()) if flips.any() else 0}

    if not want_cpu:
        return parity, None

    # ---- CPU baseline: full 100M-priority draw + gather from a host slice of the table
    sub_cap = min(cap, 4000)                      # 756 MB host slice: requests folded into it
    host_tab = table.read(0, sub_cap * table.trajectory_stride)
    path = CpuPath(rows, T, L, hp, host_tab, sub_cap, cores)
    cpu = path.time(u, steps=3, warmup=1)
    return parity, cpu


class CpuPath:
    """The path on the host cores, for timing: the prioritized draw over ALL priorities, then the
    gather.  Two draws are timed and the faster one counts: the plain one (flat float64 running
    sum over the threads + one upper_bound per variate) and the port of the two-level table (the
    GPU's addition tree in scalar C, partitions striped over the threads).  Addressing is the
    reference's own sub() compiled from its sources when that library is present, else the port;
    the bytes move by memcpy.  The table is a slice of `sub_cap` trajectories with the requests
    folded into it (the full table does not fit a bounded host sample)."""

    def __init__(self, rows, T, L, prio, host_table, sub_cap, cores):
        import numpy as np
        from oracle import oracle as O
        self.np, self.O = np, O
        self.rows, self.T, self.L, self.prio, self.tab, self.sub_cap, self.cores = rows, T, L, prio, host_table, sub_cap, cores
        self.cols = list(range(len(rows)))
        self.accu, self.stride = O.table_layout(rows, T)
        self.cdf = np.empty(len(prio), np.float32)
        self.cum = np.empty(len(prio), np.float64)
        self.ref = None
        if O.Reference.available():
            try:
                self.ref = O.Reference(rows, T, sub_cap)
                for c in self.cols:
                    self.ref.set(c, 0, L, 2)
            except Exception:      # the compiled reference is optional
                self.ref = None
        self.out = None

    def draw_plain(self, u):
        return self.O.plain_cumsum_search(self.prio, u, self.cores, scale=True, cum=self.cum)[0]

    def draw_tree(self, u):
        c2, l2, _, _ = self.O.scan_mt(self.prio, self.cores, cdf=self.cdf)
        return self.O.search(c2, l2, u, scale=True)

    def gather(self, flat):
        np, O = self.np, self.O
        B = len(flat)
        if self.out is None or len(self.out[0]) != B * self.L * self.rows[0]:
            self.out = [np.empty(B * self.L * r, np.uint8) for r in self.rows]
        i2, t2, n2 = O.decode(flat % (self.sub_cap * self.T), self.T)
        if self.ref is not None:
            self.ref.time_gather(self.tab, i2, t2, n2, self.cols, self.out, self.cores, 1)
        else:
            O.gather_mt(self.tab, self.out, i2, t2, n2, self.stride, self.T, self.accu[:len(self.rows)], self.rows,
                        [0] * len(self.rows), [self.L] * len(self.rows), [0] * len(self.rows), self.cores)

    def time(self, u, steps, warmup):
        """`steps` timed steps of each draw and of the gather after `warmup` untimed ones."""
        B = len(u)
        t = {}
        flat = None
        for name, fn in (("plain", self.draw_plain), ("tree", self.draw_tree)):
            for _ in range(warmup):
                fn(u)
            t0 = time.perf_counter()
            for _ in range(steps):
                flat = fn(u)
            t[name] = (time.perf_counter() - t0) / steps
        for _ in range(warmup):
            self.gather(flat)
        t0 = time.perf_counter()
        for _ in range(steps):
            self.gather(flat)
        t["gather"] = (time.perf_counter() - t0) / steps
        draw = min(t["plain"], t["tree"])
        step_s = draw + t["gather"]
        which = "plain float64 running sum + upper_bound" if t["plain"] <= t["tree"] else "port of the two-level table"
        addr = "reference sub() compiled from its sources" if self.ref is not None else "port of sub()"
        return {"value": B * self.L / step_s, "unit": UNIT, "cores": self.cores,
                "kind": "reference" if self.ref is not None else "port", "ms_per_step": step_s * 1e3,
                "draw_ms": {"plain_cumsum_upper_bound": t["plain"] * 1e3, "two_level_tree_port": t["tree"] * 1e3},
                "gather_ms": t["gather"] * 1e3,
                "time_share": {"draw (a port: the reference draws with torch.multinomial and has no CPU code for it)": draw / step_s,
                               f"addressing + memcpy ({addr})": t["gather"] / step_s},
                "sample": f"{steps} steps after {warmup} warm-up: draw over all {len(self.prio)} priorities on {self.cores} "
                          f"threads (the faster of two draws counts: {which}) + {B} requests gathered from a "
                          f"{self.sub_cap}-trajectory host slice of the table (requests folded into it)"}

    def close(self):
        if self.ref is not None:
            self.ref.close()
            self.ref = None


# --------------------------------------------------------------------------- #
# reference arm: the reference's CPU path on the host cores
# --------------------------------------------------------------------------- #
def run_reference(args):
    import numpy as np
    from oracle import oracle as O

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    if args.gpus == 1 and args.workload != "c5":
        cfg = C3
        rows, T, L, B, cap = cfg["rows"], cfg["T"], cfg["L"], cfg["B"], cfg["capacity"]
        n = cap * T
        config = {"workload": cfg["name"], "trajectories": cap, "trajectory_length": T, "row_bytes": rows,
                  "batch": B, "segment_length": L, "priorities": n, "table_bytes": n * sum(rows)}
    else:
        cfg = C5
        rows, T, L, B, cap = cfg["rows"], cfg["T"], cfg["L"], cfg["B_global"], cfg["capacity"]
        n = cap * T * args.gpus    # every shard's priorities, scanned by the host threads
        config = {"workload": cfg["name"], "trajectories_per_gpu": cap, "trajectory_length": T, "row_bytes": rows,
                  "global_batch": B, "batch_per_gpu": B // args.gpus, "segment_length": L,
                  "priorities_per_gpu": cap * T, "table_bytes_per_gpu": cap * T * sum(rows),
                  "parallelism": f"trajectory-id shards x{args.gpus}"}
    sub_cap = 2000
    accu, stride = O.table_layout(rows, T)
    table = np.resize(O.philox_u32(1, 0, 0, 1 << 20).view(np.uint8), sub_cap * stride)
    prio = np.resize(O.synth_lognormal(2, 0, 1 << 20), n)
    u = O.synth_u01(3, 0, B)
    path = CpuPath(rows, T, L, prio, table, sub_cap, cores)
    # Bounded: a CPU step takes tens of milliseconds, so the requested counts are honoured up to a
    # total of about 2000 step-equivalents' worth of time (they are in the thousands only for GPU runs).
    K, W = max(1, min(args.steps, 200)), max(1, min(args.warmup, 20))
    cpu = path.time(u, steps=K, warmup=W)
    path.close()
    config["l2"] = "host memory: every step streams all priorities"
    config["step"] = "draw over all priorities + addressing + memcpy gather on the host cores"
    line = {"impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": K, "warmup": W, "ms_per_step": cpu["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 / f64 sums, u8 gather", "data": "synthetic", "config": config,
            "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# the index-only and the zero-copy configurations (reported beside the headline, same line format)
# --------------------------------------------------------------------------- #
C2 = dict(name="index_sampling_only_1Mi", n=1 << 20, B=4096)
C4 = dict(name="host_zero_copy_frame_stacks_1Mstep", rows=[28224, 4, 4, 1], T=1000, capacity=1000, B=512, L=32)


def _event_loop(torch, fn, K, W):
    for i in range(W):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / K


def run_index_only(args):
    """Config 2: 1,048,576 priorities, 4096 variates U[0,total) supplied from the host: inclusive
    prefix-scan + batched binary search -> int64 indices.  The 8 MB working set stays in L2 and a
    step is two short dependent launches, so the yardstick is a latency model, not the HBM peak:
    launch + one DRAM/L2 round trip per dependent load of the step's critical path."""
    import torch
    from gear_b200 import _native as N
    from gear_b200 import core
    from oracle import oracle as O
    dev = torch.device("cuda:0"); core.init(0)
    n, B = C2["n"], C2["B"]
    hp = O.synth_lognormal(0x6EA20102, 0, n)
    prio = torch.from_numpy(hp).to(dev)
    s = core.PrioritySampler(n)
    s.scan(prio)
    total, _ = s.result()
    hu = O.synth_u01(0x6EA20202, 0, B) * total          # U[0,total) supplied from the host
    u = torch.from_numpy(hu).to(dev)
    out = torch.empty(B, dtype=torch.int64, device=dev)
    K, W = args.steps, max(args.warmup, 3)
    ms = _event_loop(torch, lambda i: s.scan_search(prio, u, scale=False, out=out), K, W)
    got_fused = out.cpu().numpy().copy()
    out.zero_()
    ms_two = _event_loop(torch, lambda i: (s.scan(prio), s.search(u, scale=False, out=out)), K, W)
    ms_scan = _event_loop(torch, lambda i: s.scan(prio), K, W)
    ms_search = _event_loop(torch, lambda i: s.search(u, scale=False, out=out), K, W)
    # end to end: the variates start in pinned host memory and the indices end there, every step
    u_host = torch.from_numpy(hu).pin_memory()
    out_host = torch.empty(B, dtype=torch.int64).pin_memory()
    Ke = max(10, min(K, 400))

    def e2e_step(i):
        u.copy_(u_host, non_blocking=True)
        s.scan_search(prio, u, scale=False, out=out)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    w0 = time.perf_counter()
    for i in range(Ke):
        e2e_step(i)
    e2e_s = (time.perf_counter() - w0) / Ke
    ocdf, ol1, _, _ = O.scan(hp)
    want, near = O.search(ocdf, ol1, hu, want_near=True)
    f64 = O.search_f64(hp, hu)
    peak, peak_src = peaks()
    scan_bytes = 8 * n + 8 * (n // 4096)
    cores = os.cpu_count() or 1
    cum = __import__("numpy").empty(n)
    reps = 20
    t0 = time.perf_counter()
    for _ in range(reps):
        c2_, l2_, _, _ = O.scan_mt(hp, cores, cdf=ocdf); O.search(c2_, l2_, hu)
    tree_s = (time.perf_counter() - t0) / reps
    t0 = time.perf_counter()
    for _ in range(reps):
        O.plain_cumsum_search(hp, hu, cores, scale=False, cum=cum)
    plain_s = (time.perf_counter() - t0) / reps
    cpu_s = min(tree_s, plain_s)
    return {
        "metric": "sampled indices/sec (prefix-scan + batched search)", "value": B / (ms * 1e-3), "unit": "indices/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 scan / f64 level-1", "data": "synthetic (seeded Philox4x32-10)",
        "config": {"workload": C2["name"], "priorities": n, "batch": B,
                   "l2": "8 MB working set: L2-resident by construction of this configuration"},
        "kernel_ms": {"scan + search in one cooperative launch (the step)": ms,
                      "the same as two launches (scan, then search behind it)": ms_two,
                      "scan alone (stores the table, builds level 1 in its last CTA)": ms_scan, "search alone": ms_search},
        "roofline": {"kernel": "scan_kernel<true>", "bound": "hbm", "achieved": scan_bytes / (ms_scan * 1e-3) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": scan_bytes / (ms_scan * 1e-3) / 1e9 / peak, "traffic": None,
                     "peak_source": peak_src, "avg_launch_ms": ms_scan, "algorithmic_bytes": scan_bytes,
                     "note": "256 partitions on 148 SMs, the data in L2: a launch- and latency-bound step, for which the "
                             "HBM fraction says little; see latency_model"},
        "latency_model": {"launch_and_drain_us_per_kernel": 2.5, "dependent_round_trip_us": 0.6,
                          "chain": "partition load, tree (two barriers), store + fence, count in, wait for all CTAs, "
                                   "aggregates into shared memory, level 1 there, variate, last entry of the partition, "
                                   "two level-2 rounds, index out: 9 trips",
                          "model_us": 2.5 + 9 * 0.6 + 1.5, "measured_us": ms * 1e3,
                          "note": "1.5 us stands for the arithmetic of the tree and of level 1 between the trips"},
        "cpu_baseline": {"value": B / cpu_s, "unit": "indices/s", "cores": cores, "kind": "port",
                         "draw_ms": {"plain_cumsum_upper_bound": plain_s * 1e3, "two_level_tree_port": tree_s * 1e3},
                         "sample": f"{reps} full steps of each draw (1,048,576 priorities + 4096 searches); the faster counts"},
        "e2e": {"value": B / e2e_s, "unit": "indices/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B,
                "ms_per_step": e2e_s * 1e3, "steps": Ke},
        "parity": {"index_mismatches_vs_oracle": int((got_fused != want).sum()),
                   "index_mismatches_vs_oracle_two_launches": int((out.cpu().numpy() != want).sum()),
                   "variates_within_1ulp_of_boundary": int(near.sum()),
                   "flips_vs_float64_running_sum": int((want != f64).sum())},
        "gpu_launches": K}


def run_zero_copy(args):
    """Config 4: the table stays in pinned, device-mapped host memory; the gather reads it over
    the host link.  Reported against the host-to-device copy peak measured in the same run."""
    import torch
    from gear_b200 import _native as N
    from gear_b200 import core
    dev = torch.device("cuda:0"); core.init(0)
    rows, T, cap, B, L = C4["rows"], C4["T"], C4["capacity"], C4["B"], C4["L"]
    table = None
    while table is None and cap >= 125:
        try:
            table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HOST)
            table.connect()
        except core.GearError:
            table, cap = None, cap // 2           # the box cannot pin that much: halve and say so
    n = cap * T
    core.fill_ptr(table.device_ptr, table.nbytes // 4, N.FILL_U32, seed=0x6EA20004)   # written over the link
    torch.cuda.synchronize()
    handler = core.StorageHandler(table)
    cols = list(range(len(rows)))
    handler.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    prio = torch.empty(n, dtype=torch.float32, device=dev)
    core.fill(prio, N.FILL_F32_LOGNORMAL, seed=0x6EA20104)
    s = core.PrioritySampler(n)
    nbatches = 8
    u = torch.empty(nbatches * B, dtype=torch.float64, device=dev)
    core.fill(u, N.FILL_U01_F64, seed=0x6EA20204)
    dsts = [torch.empty(B * L * r, dtype=torch.uint8, device=dev) for r in rows]
    flat = torch.empty(B, dtype=torch.int64, device=dev)

    def step(i):
        s.scan(prio)
        s.sample_gather(handler, u[(i % nbatches) * B:(i % nbatches + 1) * B], cols, dsts, scale=True, out_flat=flat)

    K, W = min(args.steps, 200), max(min(args.warmup, 10), 3)
    ms = _event_loop(torch, step, K, W)
    # host-link peak: best of 10 pinned H2D copies of 1 GiB
    src = torch.empty(1 << 30, dtype=torch.uint8).pin_memory(); dst = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); dst.copy_(src, non_blocking=True); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    link_gbs = (1 << 30) / (best * 1e-3) / 1e9
    gathered = B * L * sum(rows)
    # parity: the indices against the oracle, every request's bytes against the host image itself
    from oracle import oracle as O
    step(0); torch.cuda.synchronize()
    img = table.host_view()
    fl = flat.cpu().numpy(); mism = 0
    ocdf, ol1, _, _ = O.scan_mt(prio.cpu().numpy(), os.cpu_count() or 1)
    idx_mism = int((fl != O.search(ocdf, ol1, u[:B].cpu().numpy(), scale=True)).sum())
    for c, r in enumerate(rows):
        got = dsts[c].cpu().numpy(); slot = L * r
        for g in range(B):
            t_, ts = divmod(int(fl[g]), T)
            nb = min(L, T - ts) * r
            a0 = t_ * table.trajectory_stride + table.accu[c] * T + ts * r
            mism += int((got[g * slot:g * slot + nb] != img[a0:a0 + nb]).sum()) + int(got[g * slot + nb:(g + 1) * slot].any())
    achieved = gathered / (ms * 1e-3) / 1e9
    # end to end: variates from pinned host memory in, the step's indices back to the host (the
    # batch itself is consumed on the device: it is 462 MB, and it just came over the same link)
    u_host = u.cpu().pin_memory()
    ub = torch.empty(B, dtype=torch.float64, device=dev)
    flat_host = torch.empty(B, dtype=torch.int64).pin_memory()
    Ke = max(5, min(K, 50))
    w0 = time.perf_counter()
    for i in range(Ke):
        ub.copy_(u_host[(i % nbatches) * B:(i % nbatches + 1) * B], non_blocking=True)
        s.scan(prio)
        s.sample_gather(handler, ub, cols, dsts, scale=True, out_flat=flat)
        flat_host.copy_(flat, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_s = (time.perf_counter() - w0) / Ke
    # CPU path on the same host table: draw over all priorities + gather straight from the image
    cores = os.cpu_count() or 1
    path = CpuPath(rows, T, L, prio.cpu().numpy(), img, cap, cores)
    cpu = path.time(u_host[:B].numpy(), steps=3, warmup=1)
    path.close()
    return ({
        "metric": METRIC, "value": B * L / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 gather",
        "data": "synthetic (seeded Philox4x32-10, written into the mapped host table by the GPU)",
        "config": {"workload": C4["name"], "trajectories": cap, "requested_trajectories": C4["capacity"],
                   "trajectory_length": T, "row_bytes": rows, "batch": B, "segment_length": L,
                   "table_bytes": table.nbytes, "residency": "pinned mapped host memory (zero-copy)",
                   "l2": "every batch reads 462 MB of fresh host memory"},
        "gathered_gb_s": achieved,
        "roofline": {"kernel": "sample_gather_kernel", "bound": "host link", "achieved": achieved, "peak": link_gbs,
                     "unit": "GB/s", "frac": achieved / link_gbs, "traffic": None,
                     "peak_source": "best of 10 pinned 1 GiB cudaMemcpyAsync H2D in this run",
                     "algorithmic_bytes": gathered},
        "cpu_baseline": cpu,
        "e2e": {"value": B * L / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B,
                "ms_per_step": e2e_s * 1e3, "steps": Ke,
                "note": "the table itself is host memory: every step's 462 MB already cross the host link inside the kernel"},
        "parity": {"gathered_byte_mismatches": mism, "index_mismatches_vs_oracle": idx_mism, "requests_byte_checked": B},
        "gpu_launches": 2 * K})


def run_profile_case(args):
    """Small single-kernel cases for ncu captures (a few hundred MB on the device):
    `scan` / `scan_totals`: --profile-n priorities (default 40M: 320 MB of traffic, larger than L2);
    `sample_gather` / `sample_gather_lazy`: config-3 rows on a 2,000-trajectory table (378 MB), B=1024, L=64;
    `gather` / `vcopy`: the unfused gather kernels on the same table and a drawn batch;
    `search`: scan + search of the index-only configuration; `update`: 1024 changed priorities;
    `zero_copy`: the sampling kernel on a table in mapped host memory; `pull`: its sharded instance;
    `step_lazy`: scan + draw through the scan's sums + owed level-1 launch on a 6,000-trajectory table (1.1 GB)."""
    import torch
    from gear_b200 import _native as N
    from gear_b200 import core

    dev = torch.device("cuda:0")
    core.init(0)
    if args.profile in ("scan", "scan_totals"):
        n = args.profile_n
        prio = torch.empty(n, dtype=torch.float32, device=dev)
        core.fill(prio, N.FILL_F32_LOGNORMAL, seed=1)
        s = core.PrioritySampler(n)
        for _ in range(args.warmup + args.steps):
            s.scan(prio, store=args.profile == "scan")
        print(json.dumps({"profile": args.profile, "n": n, "result": s.result()}))
        return
    if args.profile == "search":
        # config 2's kernels: 1,048,576 priorities, 4096 variates
        n, B = C2["n"], C2["B"]
        prio = torch.empty(n, dtype=torch.float32, device=dev)
        core.fill(prio, N.FILL_F32_LOGNORMAL, seed=1)
        s = core.PrioritySampler(n)
        u = torch.empty(B, dtype=torch.float64, device=dev)
        core.fill(u, N.FILL_U01_F64, seed=4)
        for _ in range(args.warmup + args.steps):
            s.scan(prio)
            s.search(u, scale=True)
        print(json.dumps({"profile": args.profile, "result": s.result()}))
        return
    if args.profile == "scan_search":
        # config 2 as one cooperative launch
        n, B = C2["n"], C2["B"]
        prio = torch.empty(n, dtype=torch.float32, device=dev)
        core.fill(prio, N.FILL_F32_LOGNORMAL, seed=1)
        s = core.PrioritySampler(n)
        u = torch.empty(B, dtype=torch.float64, device=dev)
        core.fill(u, N.FILL_U01_F64, seed=4)
        for _ in range(args.warmup + args.steps):
            s.scan_search(prio, u, scale=True)
        print(json.dumps({"profile": args.profile, "result": s.result()}))
        return
    if args.profile == "zero_copy":
        # config 4's rows on a 64-trajectory table in pinned mapped host memory (1.8 GB), B=512, L=32
        rows, T, cap, B, L = C4["rows"], C4["T"], 64, C4["B"], C4["L"]
        table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HOST)
    elif args.profile == "pull":
        # the sharded instance of the sampling kernel, three shards of config 5's rows held by this one
        # GPU (the kernel is the one the ranks run; what it cannot show here is the NVLink)
        rows, T, cap, B, L = C5["rows"], C5["T"], 300, 1024, C5["L"]
        table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    else:
        # `step_lazy` needs more than 1024 partitions (level 1 is only owed for such tables): 6,000,000 priorities
        rows, T, cap, B, L = C3["rows"], C3["T"], (6000 if args.profile == "step_lazy" else 2000), C3["B"], C3["L"]
        table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    table.connect()
    fill_table(core, N, table, seed=2)
    h = core.StorageHandler(table)
    cols = list(range(len(rows)))
    h.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    n = cap * T
    prio = torch.empty(n, dtype=torch.float32, device=dev)
    core.fill(prio, N.FILL_F32_LOGNORMAL, seed=3)
    s = core.PrioritySampler(n)
    s.scan(prio, store=args.profile in ("sample_gather", "gather", "vcopy"))
    u = torch.empty(B, dtype=torch.float64, device=dev)
    core.fill(u, N.FILL_U01_F64, seed=4)
    dsts = [torch.empty(B * L * r, dtype=torch.uint8, device=dev) for r in rows]
    if args.profile in ("gather", "vcopy"):
        # the stand-ins for the reference's three copy kernels, on the indices of one draw
        flat = s.search(u, scale=True)
        idx, ts, ln = core.decode(flat, T)
        src_off, dst_off, nbytes, slot = h.sub(idx.cpu().numpy(), ts.cpu().numpy(), ln.cpu().numpy(), 0)
        so, do, nb = (torch.from_numpy(x).to(dev) for x in (src_off, dst_off, nbytes))
        for _ in range(args.warmup + args.steps):
            if args.profile == "gather":
                h.gather(cols, idx, ts, ln, dsts, zero_fill=True)
            else:
                core.vcopy(table.device_ptr, dsts[0], so, do, nb, slot)
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.profile, "requests": B, "column0_slot_bytes": int(slot)}))
        return
    if args.profile == "update":
        s.scan(prio, store=False)
        idx = (torch.arange(B, device=dev, dtype=torch.int64) * 97_003) % n
        val = torch.rand(B, device=dev, dtype=torch.float32)
        for _ in range(args.warmup + args.steps):
            s.update(prio, idx, val)
        print(json.dumps({"profile": args.profile, "result": s.result()}))
        return
    if args.profile == "pull":
        W = 3
        shards = [(table, prio, s)]
        for j in range(1, W):
            tj = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
            tj.connect()
            fill_table(core, N, tj, seed=2 + j)
            pj = torch.empty(n, dtype=torch.float32, device=dev)
            core.fill(pj, N.FILL_F32_LOGNORMAL, seed=3 + j)
            shards.append((tj, pj, core.PrioritySampler(n)))
        for tj, pj, sj in shards:
            sj.scan(pj, store=False)
        totals = torch.stack([sj.l1[-1] for _, _, sj in shards])
        us = torch.sort(u).values
        for _ in range(args.warmup + args.steps):
            s.pull(h, totals, None, [sj.l1_ptr for _, _, sj in shards], [tj.device_ptr for tj, _, _ in shards], us,
                   cols, dsts, ring=True, self_shard=0, prios=[pj.data_ptr() for _, pj, _ in shards],
                   blks=[sj.block_totals()[sj.block_totals()[2]] for _, _, sj in shards])
        print(json.dumps({"profile": args.profile, "result": s.result()}))
        return
    if args.profile == "step_lazy":
        # the headline step's three launches: scan, sampling launch that draws through the scan's sums,
        # and the level-1 launch that follows the next scan
        for _ in range(args.warmup + args.steps):
            s.scan(prio, store=False)
            s.sample_gather(h, u, cols, dsts, scale=True, zero_fill=True)
        print(json.dumps({"profile": args.profile, "result": s.result()}))
        return
    for _ in range(args.warmup + args.steps):
        s.sample_gather(h, u, cols, dsts, scale=True, zero_fill=True)
    print(json.dumps({"profile": args.profile, "result": s.result()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile", default=None,
                    choices=["scan", "scan_totals", "sample_gather", "sample_gather_lazy", "gather", "vcopy", "search",
                             "update", "zero_copy", "pull", "step_lazy", "scan_search"],
                    help="run one small single-kernel case (for ncu) instead of the benchmark")
    ap.add_argument("--workload", default="default", choices=["default", "c2", "c4", "c5"],
                    help="default: the HBM-resident table at one GPU (with c2 and c4 beside it), the sharded table at "
                         "several; c2 / c4: the index-only and zero-copy configurations alone; c5: one shard of the "
                         "sharded table on one GPU")
    ap.add_argument("--profile-n", type=int, default=40_000_000, help="priorities for --profile scan")
    args = ap.parse_args()
    if args.profile:
        return run_profile_case(args)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "c2":
        return print(json.dumps(run_index_only(args)))
    if args.workload == "c4":
        return print(json.dumps(run_zero_copy(args)))
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1 and args.workload != "c5":
        return run_ours_single(args)
    import bench_sharded
    return bench_sharded.run(args)


if __name__ == "__main__":
    main()
