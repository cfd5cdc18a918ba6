"""Multi-GPU leg of bench.py: the trajectory-id sharded token table of BASELINE.json.

Per GPU: 32,000 trajectories x 1000 steps, rows 4096/4/4 bytes (131.3 GB in HBM), one float32
priority per step.  Per step every rank rescans its priorities, the shard totals are
all-gathered, the global sorted batch of 1024 x world variates is routed, owners search +
gather in one launch into per-requester send regions, and one grouped NCCL all-to-all lands
each rank's 1024 segments of L=16 in its output tensors.  Weak scaling: per-GPU table and
per-GPU batch are fixed.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np


def run(args):
    import torch
    import torch.distributed as dist

    from . import _native as N
    from . import core
    from .comm import Communicator
    from .sharded import ShardedReplay

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
    for i in range(W_):
        replay.step_sorted(prio, batches[i % nb], batches_dev[i % nb])
    barrier()

    K = args.steps
    clocks = B.ClockSampler(local)
    if rank == 0:
        clocks.start()
        time.sleep(0.12)
    scan_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    e0.record()
    for i in range(K):
        scan_ev[i][0].record()
        replay.scan(prio)
        scan_ev[i][1].record()
        replay.step_sorted(prio, batches[i % nb], batches_dev[i % nb], rescan=False)
    e1.record()
    barrier()
    t1 = time.time()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    scan_ms = torch.tensor([sum(a.elapsed_time(c) for a, c in scan_ev) / K], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(scan_ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms[0]) / K
    clk = clocks.stop(t0, t1) if rank == 0 else None

    # ---- end to end: the rank's slice goes back to pinned host memory every step
    slots = [L * r for r in rows]
    out_host = [torch.empty(b * s, dtype=torch.uint8).pin_memory() for s in slots]
    idx_host = torch.empty(b, dtype=torch.int64).pin_memory()
    Ke = max(5, min(K, 100))
    barrier()
    w0 = time.perf_counter()
    for i in range(Ke):
        colsout, gflat = replay.step(prio, batches[i % nb])       # variates start on the host here
        for h, d in zip(out_host, colsout):
            h.copy_(d, non_blocking=True)
        idx_host.copy_(gflat, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    barrier()
    e2e_s = torch.tensor([(time.perf_counter() - w0) / Ke], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)

    # ---- parity of one batch: indices against the oracle on all shards' priorities, bytes of
    #      locally owned requests against read-backs of the table
    parity = sharded_parity(replay, table, handler, prio, batches[0], rank, world, dev, T, rows, L, b)

    if rank == 0:
        gathered = b * sum(slots)                      # per rank
        peak, peak_src = B.peaks()
        scan_bytes = 8 * n_local + 8 * ((n_local + 4095) // 4096)
        achieved = scan_bytes / (float(scan_ms[0]) * 1e-3) / 1e9
        line = {
            "metric": B.METRIC, "value": Bg * L / (ms_step * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": K,
            "warmup": W_, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 scan / f64 level-1 / u8 gather", "data": "synthetic (seeded Philox4x32-10, generated in HBM)",
            "config": {"workload": cfg["name"], "trajectories_per_gpu": cap, "trajectory_length": T, "row_bytes": rows,
                       "batch_per_gpu": b, "global_batch": Bg, "segment_length": L, "priorities_per_gpu": n_local,
                       "table_bytes_per_gpu": table.nbytes, "parallelism": f"trajectory-id shards x{world}",
                       "l2": "inputs larger than L2 (128 MB of priorities re-read every step per GPU)",
                       "step": "scan + all-gather totals + route + search/gather + all-to-all"},
            "gathered_gb_s": 2 * gathered * world / (ms_step * 1e-3) / 1e9,
            "exchanged_bytes_per_step_per_gpu": int(gathered * (world - 1) / world),
            "roofline": {"kernel": "scan_kernel", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes": scan_bytes, "avg_launch_ms": float(scan_ms[0])},
            "cpu_baseline": None,
            "e2e": {"value": Bg * L / float(e2e_s[0]), "unit": B.UNIT, "h2d_bytes_per_step": 8 * Bg * world,
                    "d2h_bytes_per_step": (gathered + 8 * b) * world, "ms_per_step": float(e2e_s[0]) * 1e3, "steps": Ke},
            "gpu_launches": 2 * K * world, "clocks": clk, "parity": parity,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sharded_parity(replay, table, handler, prio, u_sorted, rank, world, dev, T, rows, L, b):
    import torch
    import torch.distributed as dist
    n_local = prio.numel()
    colsout, gflat = replay.step_sorted(prio, u_sorted, torch.from_numpy(u_sorted).to(dev))
    torch.cuda.synchronize()
    gflat_h = gflat.cpu().numpy()
    plan = replay.last_plan
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
    mism = torch.tensor([byte_mismatch, checked], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(mism)
    out = None
    if rank == 0:
        # The sharded draw is defined shard by shard: each shard's own cumulative table, shard
        # totals summed in rank order, then the owner-local search.  (It coincides with one table
        # over the concatenated priorities only when a shard holds a whole number of partitions.)
        from oracle import oracle as O
        from .sharded import route
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
    return out
