"""Multi-GPU leg of bench.py: the trajectory-id sharded token table of BASELINE.json.

Per GPU: 32,000 trajectories x 1000 steps, rows 4096/4/4 bytes (131.3 GB in HBM), one float32
priority per step.  Two ways of moving the segments are timed on the same table and batches:
* all-to-all: every rank rescans its priorities, the shard totals are all-gathered, the global
  sorted batch of 1024 x world variates is routed on the host, owners search + gather in one
  launch into per-requester send regions, and one grouped NCCL all-to-all lands each rank's 1024
  segments of L=16 in its output tensors;
* pull (the headline): after the scan and the all-gather of the totals, each rank's single launch
  routes its 1024 requests, searches the owners' cumulative tables and copies the segments out of
  the owners' HBM over NVLink.
Weak scaling: per-GPU table and per-GPU batch are fixed.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np


def run(args):
    import torch
    import torch.distributed as dist

    from gear_b200 import _native as N
    from gear_b200 import core
    from gear_b200.comm import Communicator
    from gear_b200.sharded import ShardedReplay

    import bench as B  # the top-level script: shared constants and helpers

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    core.init(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator.from_torch_distributed()
    else:
        comm = None

    cfg = B.C5
    rows, T, cap, L, b = cfg["rows"], cfg["T"], cfg["capacity"], cfg["L"], cfg["B_per_rank"]
    if os.environ.get("GEAR_BENCH_SMALL"):   # smoke-sized shard for functional runs
        cap = 2000
    n_local = cap * T
    Bg = b * world
    cols = list(range(len(rows)))

    table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    table.connect()
    core.fill_ptr(table.device_ptr, table.nbytes // 4, N.FILL_I32_RANGE, seed=0x6EA20005 + rank, a=0, b=50257)
    handler = core.StorageHandler(table)
    handler.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    prio = torch.empty(n_local, dtype=torch.float32, device=dev)
    core.fill(prio, N.FILL_F32_LOGNORMAL, seed=0x6EA20105 + rank)
    sampler = core.PrioritySampler(n_local)
    replay = ShardedReplay(handler, sampler, cols, rank, world, comm, max_global_batch=Bg)

    # the same sorted global batches on every rank (counter-based generator, same key)
    nb = 8
    rng = np.random.Generator(np.random.Philox(key=0x6EA20205))
    batches = [np.sort(rng.random(Bg)) for _ in range(nb)]
    batches_dev = [torch.from_numpy(x).to(dev) for x in batches]   # resident before the clock starts

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    W_ = max(args.warmup, 3)
    K = args.steps
    clocks = B.ClockSampler(local)

    def timed(step, sample_clocks):
        """W_ warm-up steps, then K timed ones between one pair of events, then an instrumented run
        with an event pair around every scan (events inside the step cost some overlap between
        launches, so they stay out of the step time): (ms per step, ms per scan, clock record),
        each the max over ranks."""
        for i in range(W_):
            step(i, True)
        barrier()
        if sample_clocks and rank == 0:
            clocks.start()
            time.sleep(0.12)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.time()
        e0.record()
        for i in range(K):
            step(i, True)
        e1.record()
        barrier()
        t1 = time.time()
        clk = clocks.stop(t0, t1) if (sample_clocks and rank == 0) else None
        Ki = min(K, 100)
        scan_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(Ki)]
        for i in range(Ki):
            scan_ev[i][0].record()
            replay.scan_for_step(scan_ev[i][1].record)   # second event right behind scan_kernel, before level 1
            step(i, False)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / K, sum(a.elapsed_time(c) for a, c in scan_ev) / Ki],
                          dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms[0]), float(ms[1]), clk

    # One GPU alone on the same shard and per-GPU batch (no peers, no collective): the number the
    # multi-GPU values are to be compared with for weak scaling.
    solo_ms = None
    if world > 1:
        full = replay
        solo_u = [x[rank::world].contiguous() for x in batches_dev]
        replay = ShardedReplay(handler, sampler, cols, 0, 1, None, max_global_batch=b)
        replay.enable_pull(double_buffer=True, ring=False)
        replay.scan_for_step = lambda mid: replay.pull_scan(prio, between=mid)
        solo_ms, _, _ = timed(lambda i, rescan: replay.step_pull(prio, solo_u[i % nb], rescan=rescan), False)
        replay.disable_pull()
        replay = full

    # mode 1: owners search + gather into send regions, one grouped NCCL all-to-all per step
    replay.scan_for_step = lambda mid: (replay.sampler.scan_partitions(prio, store=True), mid(),
                                        replay.sampler.scan_level1())
    a2a_ms, a2a_scan_ms, clk_a2a = timed(
        lambda i, rescan: replay.step_sorted(prio, batches[i % nb], batches_dev[i % nb], rescan=rescan),
        sample_clocks=False)
    parity_a2a = sharded_parity(replay, table, handler, prio, batches[0], rank, world, dev, T, rows, L, b, "alltoall")

    # mode 2: no exchange step -- requesters read the owners' HBM in place over NVLink
    ring = os.environ.get("GEAR_BENCH_PULL_RING", "1") != "0"      # tuning knob; rings are the default
    replay.enable_pull(double_buffer=True, ring=ring, mailbox=os.environ.get("GEAR_BENCH_PULL_MAILBOX", "1") != "0")
    replay.scan_for_step = lambda mid: replay.pull_scan(prio, between=mid)
    pull_ms, pull_scan_ms, clk = timed(
        lambda i, rescan: replay.step_pull(prio, batches_dev[i % nb], rescan=rescan), sample_clocks=True)
    parity = sharded_parity(replay, table, handler, prio, batches[0], rank, world, dev, T, rows, L, b, "pull")
    ms_step, scan_ms = pull_ms, pull_scan_ms

    # ---- end to end: the rank's slice goes back to pinned host memory every step
    slots = [L * r for r in rows]
    out_host = [torch.empty(b * s, dtype=torch.uint8).pin_memory() for s in slots]
    idx_host = torch.empty(b, dtype=torch.int64).pin_memory()
    u_host = [torch.from_numpy(x).pin_memory() for x in batches]
    u_dev = torch.empty(Bg, dtype=torch.float64, device=dev)
    Ke = max(5, min(K, 100))
    barrier()
    w0 = time.perf_counter()
    for i in range(Ke):
        u_dev.copy_(u_host[i % nb], non_blocking=True)            # variates start on the host here
        colsout, gflat = replay.step_pull(prio, u_dev)
        for h, d in zip(out_host, colsout):
            h.copy_(d, non_blocking=True)
        idx_host.copy_(gflat, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    barrier()
    e2e_s = torch.tensor([(time.perf_counter() - w0) / Ke], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)

    replay.disable_pull()
    if rank == 0:
        gathered = b * sum(slots)                      # per rank
        peak, peak_src = B.peaks()
        scan_bytes = 8 * n_local + 8 * ((n_local + 4095) // 4096)
        achieved = scan_bytes / (scan_ms * 1e-3) / 1e9
        line = {
            "metric": B.METRIC, "value": Bg * L / (ms_step * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": K,
            "warmup": W_, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 scan / f64 level-1 / u8 gather", "data": "synthetic (seeded Philox4x32-10, generated in HBM)",
            "config": {"workload": cfg["name"], "trajectories_per_gpu": cap, "trajectory_length": T, "row_bytes": rows,
                       "batch_per_gpu": b, "global_batch": Bg, "segment_length": L, "priorities_per_gpu": n_local,
                       "table_bytes_per_gpu": table.nbytes, "parallelism": f"trajectory-id shards x{world}",
                       "l2": "inputs larger than L2 (128 MB of priorities re-read every step per GPU)",
                       "step": "scan + level 1 + shard totals written into every rank's mailbox + one launch that "
                               "routes, searches and gathers from the owners' HBM over NVLink (no collective)"},
            "exchange_modes": {
                "pull_over_nvlink": {"ms_per_step": pull_ms, "value": Bg * L / (pull_ms * 1e-3), "parity": parity},
                "nccl_alltoall": {"ms_per_step": a2a_ms, "value": Bg * L / (a2a_ms * 1e-3), "parity": parity_a2a,
                                  "step": "scan + all-gather totals + host routing + owner search/gather + "
                                          "grouped ncclSend/ncclRecv all-to-all"}},
            "one_gpu_same_workload": None if solo_ms is None else {
                "ms_per_step": solo_ms, "value": b * L / (solo_ms * 1e-3), "unit": B.UNIT,
                "note": "each GPU alone on its own shard with the same per-GPU batch, max over ranks"},
            "gathered_gb_s": 2 * gathered * world / (ms_step * 1e-3) / 1e9,
            "exchanged_bytes_per_step_per_gpu": int(gathered * (world - 1) / world),
            "roofline": {"kernel": "scan_kernel<true>", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes": scan_bytes, "avg_launch_ms": scan_ms},
            "cpu_baseline": None,
            "e2e": {"value": Bg * L / float(e2e_s[0]), "unit": B.UNIT, "h2d_bytes_per_step": 8 * Bg * world,
                    "d2h_bytes_per_step": (gathered + 8 * b) * world, "ms_per_step": float(e2e_s[0]) * 1e3, "steps": Ke},
            "gpu_launches": 3 * K * world, "clocks": clk, "parity": parity,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sharded_parity(replay, table, handler, prio, u_sorted, rank, world, dev, T, rows, L, b, mode):
    """Parity of one batch: indices of every rank's slice against the oracle on all shards'
    priorities; bytes of the requests this rank owns itself against read-backs of its table; in
    pull mode additionally every byte of the slice against the all-to-all mode's result."""
    import torch
    import torch.distributed as dist
    from gear_b200.sharded import plan_sorted
    n_local = prio.numel()
    cross = None
    if mode == "pull":
        ref_cols, ref_flat = replay.step_sorted(prio, u_sorted, torch.from_numpy(u_sorted).to(dev))
        ref_cols, ref_flat = [c.clone() for c in ref_cols], ref_flat.clone()
        colsout, gflat = replay.step_pull(prio, torch.from_numpy(u_sorted).to(dev))
        torch.cuda.synchronize()
        cross = sum(int((a != c).sum()) for a, c in zip(ref_cols, colsout)) + int((ref_flat != gflat).sum())
        del ref_cols
        plan, _, _ = plan_sorted(replay.gather_totals(), u_sorted, rank, world)
    else:
        colsout, gflat = replay.step_sorted(prio, u_sorted, torch.from_numpy(u_sorted).to(dev))
        torch.cuda.synchronize()
        plan = replay.last_plan
    gflat_h = gflat.cpu().numpy()
    # bytes: requests of my slice that I own myself, against table read-backs
    byte_mismatch = checked = 0
    own = np.nonzero(plan.slice_owner == rank)[0][::8]
    for c, r in enumerate(rows):
        got = colsout[c].cpu().numpy()
        slot = L * r
        for s in own:
            fl = int(gflat_h[s]) - rank * n_local
            t, ts = divmod(fl, T)
            nb = min(L, T - ts) * r
            src = t * table.trajectory_stride + table.accu[c] * T + ts * r
            want = table.read(src, nb)
            byte_mismatch += int((got[s * slot:s * slot + nb] != want).sum()) + int(got[s * slot + nb:(s + 1) * slot].any())
            checked += 1
    # indices: every rank's slice against the oracle on the concatenated priorities (rank 0 computes)
    allp = [torch.empty_like(prio) for _ in range(world)] if world > 1 else [prio]
    allf = [torch.empty_like(gflat) for _ in range(world)] if world > 1 else [gflat]
    if world > 1:
        dist.all_gather(allp, prio)
        dist.all_gather(allf, gflat.contiguous())
    mism = torch.tensor([byte_mismatch, checked, cross or 0], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(mism)
    out = None
    if rank == 0:
        # The sharded draw is defined shard by shard: each shard's own cumulative table, shard
        # totals summed in rank order, then the owner-local search.  (It coincides with one table
        # over the concatenated priorities only when a shard holds a whole number of partitions.)
        from oracle import oracle as O
        from gear_b200.sharded import route
        scans = [O.scan_mt(p.cpu().numpy(), os.cpu_count() or 1) for p in allp]
        totals = np.array([sc[2] for sc in scans])
        owner, residual, _ = route(totals, u_sorted, world)
        want = np.empty(len(u_sorted), np.int64)
        for j in range(world):
            m = owner == j
            want[m] = O.search(scans[j][0], scans[j][1], residual[m]) + j * n_local
        got = torch.cat(allf).cpu().numpy()
        out = {"index_mismatches_vs_oracle": int((got != want).sum()), "gathered_byte_mismatches": int(mism[0]),
               "requests_byte_checked": int(mism[1])}
        if mode == "pull":
            out["mismatches_vs_alltoall_mode_all_bytes"] = int(mism[2])
    return out
