"""Multi-GPU leg of bench.py: the trajectory-id sharded token table (config 5 of the benchmark set).

Per GPU: 32,000 trajectories x 1000 steps, rows 4096/4/4 bytes (131.3 GB in HBM), one float32
priority per step.  The global batch is 8192 requests of L=16 at every number of GPUs (each rank
consumes 8192 / N of them); a second batch size, 1024 per rank, is timed beside it.  Two ways of
moving the segments, on the same table and batches:
* pull (the headline): totals-only scan, level 1, then every rank writes its level 1 and total
  into its peers' mailboxes and ONE launch per rank routes its requests, searches and copies the
  segments out of the owners' HBM over NVLink -- no collective, no host synchronisation;
* all-to-all: scan, all-gather of the shard totals (one host synchronisation: NCCL needs the
  message sizes), owners search + gather into per-requester send regions, one grouped NCCL
  all-to-all into the requesters' final tensors.
Two ways of dealing the sorted batch to the ranks: contiguous slices (the reference's partition;
nearly every request then lands on the requester's own shard) and scattered (rank r takes requests
r, r+N, ...: (N-1)/N of a rank's requests are remote, which is what measures the exchange).
Remote requests and bytes are counted from the sampled ids, never derived from a formula.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np


def _small_oracle_case(rank, world, comm, dev):
    """Every byte and index of small batches against the CPU oracle's single-process gather from the
    concatenated table: both exchange modes, both layouts, a batch that lands on shard 0 alone."""
    import torch
    from gear_b200 import _native as N
    from gear_b200 import core
    from gear_b200.sharded import ShardedReplay
    from oracle import oracle as O

    rows, T, cap, L, b = [4096, 4, 12, 1], 64, 128, 16, 96
    n_local, B = cap * T, b * world
    cols = list(range(len(rows)))

    def shard_data(r):
        accu, stride = O.table_layout(rows, T)
        img = O.philox_u32(100 + r, 0, 0, (stride * cap + 3) // 4).view(np.uint8)[: stride * cap].copy()
        prio = O.synth_lognormal(200 + r, 0, n_local)
        prio[r::5] = 0.0
        return img, prio

    img, prio = shard_data(rank)
    table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    table.connect()
    table.write(0, img)
    handler = core.StorageHandler(table)
    handler.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    sampler = core.PrioritySampler(n_local)
    pbuf = core.DeviceBuffer(n_local * 4)
    dprio = pbuf.view(torch.float32)
    dprio.copy_(torch.from_numpy(prio))
    imgs, prios = zip(*[shard_data(r) for r in range(world)])
    gimg, gprio = np.concatenate(imgs), np.concatenate(prios)
    gcdf, gl1, _, _ = O.scan(gprio)               # shards are whole partitions: one table over all of them
    accu, stride = O.table_layout(rows, T)
    replay = ShardedReplay(handler, sampler, cols, rank, world, comm, max_global_batch=B, store=False)
    replay.enable_pull(ring=True, priorities=pbuf)
    bad = checked = 0
    for trial in range(3):
        u01 = np.sort(O.synth_u01(300 + trial, 0, B))
        if trial == 2:
            u01[:] = np.sort(O.synth_u01(400, 0, B) * 0.01)     # every request lands on shard 0
        du = torch.from_numpy(u01).to(dev)
        want_all = O.search(gcdf, gl1, u01, scale=True)
        for layout in ("contiguous", "scattered"):
            want_flat = want_all[rank * b:(rank + 1) * b] if layout == "contiguous" else want_all[rank::world]
            gi, gt, gl = O.decode(want_flat, T)
            for mode in ("pull", "alltoall"):
                if mode == "pull":
                    outs, gflat = replay.step_pull(dprio, du, layout=layout)
                else:
                    outs, gflat = replay.step_sorted(dprio, u01, du, layout=layout)
                torch.cuda.synchronize()
                bad += int((gflat.cpu().numpy() != want_flat).sum())
                for c in cols:
                    want = O.fused_subcopy(gimg, gi, gt, gl, stride, int(accu[c]), T, rows[c], 0, L, False)
                    bad += int((outs[c].cpu().numpy() != want).sum())
                checked += 1
    st = sampler.result()[1][0]
    replay.disable_pull()
    t = torch.tensor([bad, checked, st], dtype=torch.int64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t)
    return {"mismatches_vs_oracle_all_bytes_and_indices": int(t[0]), "batches_checked": int(t[1]),
            "status_bits": int(t[2]), "case": f"{world} shards of {n_local} steps, {B} requests, rows {rows}, "
            "both exchange modes x both layouts x 3 batches (one of them entirely on shard 0)"}


def run(args, emit=True):
    """emit=False (one process, one GPU): return the line instead of printing it."""
    import torch
    import torch.distributed as dist

    from gear_b200 import _native as N
    from gear_b200 import core
    from gear_b200.comm import Communicator
    from gear_b200.sharded import ShardedReplay, requester_of

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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allmax(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def allsum(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t)
        return [float(x) for x in t]

    small = _small_oracle_case(rank, world, comm, dev)

    cfg = B.C5
    rows, T, cap, L = cfg["rows"], cfg["T"], cfg["capacity"], cfg["L"]
    if os.environ.get("GEAR_BENCH_SMALL"):   # smoke-sized shard for functional runs
        cap = 2000
    n_local = cap * T
    cols = list(range(len(rows)))
    slots = [L * r for r in rows]
    Bg_main = cfg["B_global"]
    Bg_side = cfg["B_per_rank"] * world
    maxB = max(Bg_main, Bg_side)

    table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    table.connect()
    core.fill_ptr(table.device_ptr, table.nbytes // 4, N.FILL_I32_RANGE, seed=0x6EA20005 + rank, a=0, b=50257)
    handler = core.StorageHandler(table)
    handler.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    pbuf = core.DeviceBuffer(n_local * 4)    # its own allocation: the peers map it
    prio = pbuf.view(torch.float32)
    core.fill(prio, N.FILL_F32_LOGNORMAL, seed=0x6EA20105 + rank)
    sampler = core.PrioritySampler(n_local)
    replay = ShardedReplay(handler, sampler, cols, rank, world, comm, max_global_batch=maxB, store=False)

    # the same sorted global batches on every rank (counter-based generator, same key)
    nb = 8
    rng = np.random.Generator(np.random.Philox(key=0x6EA20205))
    batches = {Bg: [np.sort(rng.random(Bg)) for _ in range(nb)] for Bg in sorted({Bg_main, Bg_side})}
    batches_dev = {Bg: [torch.from_numpy(x).to(dev) for x in v] for Bg, v in batches.items()}   # resident before the clock starts

    W_ = max(args.warmup, 3)
    K = args.steps
    clocks = B.ClockSampler(local)

    spin_steps = 300      # 50-80 ms of steps on this configuration: a clock sample or two (every 50 ms) fall into them

    def timed(step, scan_only, sample_clocks=False):
        """W_ warm-up steps, then K timed ones between one pair of events; then an instrumented run of
        the same steps with events after the scan's first launch, after level 1 and at the end of the
        step (events inside a step cost some overlap between launches, so they stay out of the step
        time).  Returns max over ranks of (ms per step, ms per scan launch, ms from the end of level 1
        to the end of the step -- the publish + pull launches, or the exchange), and the clock record."""
        # The clock sampler starts first, and 50-80 ms of the same steps (untimed, a fixed count agreed by
        # all ranks) bring the GPUs from idle to their working clocks before the warm-up steps proper.
        if sample_clocks and rank == 0:
            clocks.start()
        barrier()
        t_load = time.time()
        for i in range(spin_steps if sample_clocks else 64):
            step(i, True)
            if i % 32 == 31:
                torch.cuda.synchronize()
        for i in range(W_):
            step(i, True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.time()
        e0.record()
        for i in range(K):
            step(i, True)
        e1.record()
        barrier()
        t1 = time.time()
        clk = clocks.stop(t_load, t1) if (sample_clocks and rank == 0) else None
        barrier()     # rank 0 spent a moment with the clock sampler: the ranks start the next loop together
        Ki = min(K, 100)
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(Ki)]
        for i in range(Ki):
            ev[i][0].record()
            scan_only(ev[i][1].record)      # event right behind scan_kernel, before level 1
            ev[i][2].record()
            step(i, False)
            ev[i][3].record()
        barrier()
        ms, scan_ms, rest_ms = allmax([e0.elapsed_time(e1) / K, sum(e[0].elapsed_time(e[1]) for e in ev) / Ki,
                                       sum(e[2].elapsed_time(e[3]) for e in ev) / Ki])
        return ms, scan_ms, rest_ms, clk

    def two_launch_scan(mid):
        sampler.scan_partitions(prio, store=False)
        mid()
        sampler.scan_level1()

    def remote_counts(gflat_list, b):
        """Remote requests and payload bytes of this rank's slices, counted from the sampled ids."""
        req = byt = 0
        for gf in gflat_list:
            g = gf.cpu().numpy()
            own = g // n_local
            ts = (g % n_local) % T
            valid = np.minimum(L, T - ts)
            m = own != rank
            req += int(m.sum())
            byt += int((valid[m] * sum(rows)).sum())
        return req, byt

    results = {}
    ring = os.environ.get("GEAR_BENCH_PULL_RING", "1") != "0"      # tuning knob; rings are the default
    # tuning knob: level 1 copied into the peers' mailboxes ("1"), searched remotely ("0"), or by layout
    copy_l1 = {"0": False, "1": True}.get(os.environ.get("GEAR_BENCH_PULL_L1COPY", "auto"), "auto")
    clk_main = None
    for Bg in sorted({Bg_main, Bg_side}, reverse=True):
        b = Bg // world
        per = {}
        # one GPU alone on its own shard with the same per-GPU batch (no peers, no collective)
        solo_ms = None
        if world > 1:
            solo = ShardedReplay(handler, sampler, cols, 0, 1, None, max_global_batch=b, store=False)
            solo.enable_pull(ring=False, priorities=pbuf)
            solo_u = [x[rank::world].contiguous() for x in batches_dev[Bg]]
            solo_ms, _, _, _ = timed(lambda i, rescan: solo.step_pull(prio, solo_u[i % nb], rescan=rescan),
                                     lambda mid: solo.pull_scan(prio, between=mid))
            solo.disable_pull()
        for layout in ("contiguous", "scattered"):
            # all-to-all mode
            a2a_ms, a2a_scan_ms, a2a_rest_ms, _ = timed(
                lambda i, rescan: replay.step_sorted(prio, batches[Bg][i % nb], batches_dev[Bg][i % nb], rescan=rescan,
                                                     layout=layout), two_launch_scan)
            par_a2a = sharded_parity(replay, table, prio, batches[Bg][0], rank, world, dev, T, rows, L, "alltoall", layout)
            # pull mode
            replay.enable_pull(ring=ring, priorities=pbuf, copy_l1=copy_l1)
            pull_ms, scan_ms, pull_rest_ms, clk = timed(
                lambda i, rescan: replay.step_pull(prio, batches_dev[Bg][i % nb], rescan=rescan, layout=layout),
                lambda mid: replay.pull_scan(prio, between=mid), sample_clocks=(Bg == Bg_main and layout == "contiguous"))
            if clk is not None:
                clk_main = clk
            flats = []
            for i in range(nb):
                _, gf = replay.step_pull(prio, batches_dev[Bg][i], layout=layout)
                flats.append(gf.clone())
            torch.cuda.synchronize()
            rreq, rbyt = remote_counts(flats, b)
            rreq_all, rbyt_all = allsum([rreq, rbyt])
            par_pull = sharded_parity(replay, table, prio, batches[Bg][0], rank, world, dev, T, rows, L, "pull", layout)
            replay.disable_pull()
            remote_b_gpu = rbyt_all / nb / world
            per[layout] = {
                "pull_over_nvlink": {
                    "ms_per_step": pull_ms, "value": Bg * L / (pull_ms * 1e-3), "scan_launch_ms": scan_ms,
                    "publish_and_pull_launch_ms": pull_rest_ms,
                    "nvlink_gb_s_per_gpu_inbound": remote_b_gpu / (pull_rest_ms * 1e-3) / 1e9,
                    "nvlink_frac_of_900_gb_s": remote_b_gpu / (pull_rest_ms * 1e-3) / 1e9 / 900.0,
                    "parity": par_pull},
                "nccl_alltoall": {
                    "ms_per_step": a2a_ms, "value": Bg * L / (a2a_ms * 1e-3), "scan_launch_ms": a2a_scan_ms,
                    "exchange_ms_after_level1": a2a_rest_ms,
                    "nvlink_gb_s_per_gpu_inbound": remote_b_gpu / (a2a_rest_ms * 1e-3) / 1e9, "parity": par_a2a},
                "remote_requests_counted_per_step": rreq_all / nb, "remote_fraction_of_requests": rreq_all / nb / Bg,
                "remote_bytes_counted_per_step_per_gpu": remote_b_gpu,
            }
        per["one_gpu_same_workload"] = None if solo_ms is None else {
            "ms_per_step": solo_ms, "value": b * L / (solo_ms * 1e-3), "unit": B.UNIT,
            "note": "each GPU alone on its own shard with the same per-GPU batch, max over ranks"}
        if solo_ms is not None:
            for layout in ("contiguous", "scattered"):
                per[layout]["pull_over_nvlink"]["efficiency_vs_one_gpu_same_workload"] = solo_ms / per[layout]["pull_over_nvlink"]["ms_per_step"]
                per[layout]["nccl_alltoall"]["efficiency_vs_one_gpu_same_workload"] = solo_ms / per[layout]["nccl_alltoall"]["ms_per_step"]
        results[Bg] = per

    # ---- end to end: the rank's slice goes back to pinned host memory every step, two batches in
    #      flight (the copy-out of a batch overlaps the next step); and the floor it is up against:
    #      all ranks copying a slice to pinned memory at once with nothing else running.
    Bg = Bg_main
    b = Bg // world
    gathered = b * sum(slots)                      # per rank
    replay.enable_pull(ring=ring, priorities=pbuf, copy_l1=copy_l1)
    depth = 2
    out_dev = [[torch.empty(b * s, dtype=torch.uint8, device=dev) for s in slots] for _ in range(depth)]
    idx_dev = [torch.empty(b, dtype=torch.int64, device=dev) for _ in range(depth)]
    out_host = [[torch.empty(b * s, dtype=torch.uint8).pin_memory() for s in slots] for _ in range(depth)]
    idx_host = [torch.empty(b, dtype=torch.int64).pin_memory() for _ in range(depth)]
    u_host = [torch.from_numpy(x).pin_memory() for x in batches[Bg]]
    u_dev = [torch.empty(Bg, dtype=torch.float64, device=dev) for _ in range(depth)]
    copy_stream = torch.cuda.Stream(device=dev)
    done = [torch.cuda.Event() for _ in range(depth)]
    ready = [torch.cuda.Event() for _ in range(depth)]
    main = torch.cuda.current_stream()

    def e2e_loop(Ke):
        for i in range(Ke):
            k = i % depth
            if i >= depth:
                done[k].synchronize()              # the caller holds batch i - depth in host memory here
            u_dev[k].copy_(u_host[i % nb], non_blocking=True)            # variates start on the host
            replay.step_pull(prio, u_dev[k], layout="contiguous", out=(out_dev[k], idx_dev[k]))
            ready[k].record(main)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ready[k])
                for h, d in zip(out_host[k], out_dev[k]):
                    h.copy_(d, non_blocking=True)
                idx_host[k].copy_(idx_dev[k], non_blocking=True)
                done[k].record(copy_stream)
        for k in range(depth):
            done[k].synchronize()

    Ke = max(6, min(K, 100))
    e2e_loop(4)
    barrier()
    w0 = time.perf_counter()
    e2e_loop(Ke)
    barrier()
    e2e_s = allmax([(time.perf_counter() - w0) / Ke])[0]
    # the last batch in host memory against the device-side result of the same variates
    kl = (Ke - 1) % depth
    colsout, gflat = replay.step_pull(prio, batches_dev[Bg][(Ke - 1) % nb], layout="contiguous")
    torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(idx_host[kl], gflat.cpu()) and all(torch.equal(h, d.cpu()) for h, d in zip(out_host[kl], colsout)))
    # D2H floor
    barrier()
    w0 = time.perf_counter()
    for i in range(Ke):
        for h, d in zip(out_host[0], out_dev[0]):
            h.copy_(d, non_blocking=True)
        idx_host[0].copy_(idx_dev[0], non_blocking=True)
    torch.cuda.synchronize()
    barrier()
    floor_s = allmax([(time.perf_counter() - w0) / Ke])[0]
    e2e_ok_all = allsum([0.0 if e2e_ok else 1.0])[0] == 0.0
    replay.disable_pull()

    if rank == 0:
        peak, peak_src = B.peaks()
        main_res = results[Bg_main]
        head = main_res["contiguous"]["pull_over_nvlink"]
        ms_step, scan_ms = head["ms_per_step"], head["scan_launch_ms"]
        scan_bytes = 4 * n_local + 8 * ((n_local + 4095) // 4096)
        achieved = scan_bytes / (scan_ms * 1e-3) / 1e9
        solo = main_res["one_gpu_same_workload"]
        line = {
            "metric": B.METRIC, "value": Bg_main * L / (ms_step * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": K,
            "warmup": W_, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 scan / f64 level-1 / u8 gather", "data": "synthetic (seeded Philox4x32-10, generated in HBM)",
            "config": {"workload": cfg["name"], "trajectories_per_gpu": cap, "trajectory_length": T, "row_bytes": rows,
                       "global_batch": Bg_main, "batch_per_gpu": Bg_main // world, "segment_length": L,
                       "priorities_per_gpu": n_local, "table_bytes_per_gpu": table.nbytes,
                       "parallelism": f"trajectory-id shards x{world}", "slice_layout": "contiguous (the reference's partition)",
                       "l2": "inputs larger than L2 (128 MB of priorities re-read every step per GPU)",
                       "step": "totals-only scan + level-1 launch that also writes the shard total and the step's number into "
                               "every rank's mailbox + one launch that routes, searches and gathers from the owners' HBM "
                               "over NVLink (no collective)"},
            "efficiency_vs_one_gpu_same_workload": None if solo is None else solo["ms_per_step"] / ms_step,
            "global_batch_8192": main_res,
            "global_batch_1024_per_gpu": results[Bg_side],
            "exchange_headline": {"slice_layout": "scattered", **main_res["scattered"]["pull_over_nvlink"],
                                  "remote_bytes_counted_per_step_per_gpu": main_res["scattered"]["remote_bytes_counted_per_step_per_gpu"],
                                  "remote_fraction_of_requests": main_res["scattered"]["remote_fraction_of_requests"]},
            "small_case_every_byte_vs_oracle": small,
            "gathered_gb_s": 2 * gathered * world / (ms_step * 1e-3) / 1e9,
            "remote_bytes_counted_per_step_per_gpu": main_res["contiguous"]["remote_bytes_counted_per_step_per_gpu"],
            "roofline": {"kernel": "scan_kernel<false> (totals only)", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes": scan_bytes, "avg_launch_ms": scan_ms,
                         "note": "the launch before every scan is a gather that has just written a batch larger than "
                                 "L2: while the scan reads its 128 MB, about as many bytes of that batch are still being "
                                 "written back from L2, so DRAM carries roughly twice the algorithmic bytes (back to "
                                 "back on a quiet GPU the same scan takes 27 us)"},
            "cpu_baseline": None,
            "e2e": {"value": Bg_main * L / e2e_s, "unit": B.UNIT, "h2d_bytes_per_step": 8 * Bg_main * world,
                    "d2h_bytes_per_step": (gathered + 8 * b) * world, "ms_per_step": e2e_s * 1e3, "steps": Ke,
                    "batches_in_flight": depth, "matches_device_result": e2e_ok_all,
                    "d2h_floor_ms_per_step": floor_s * 1e3, "frac_of_d2h_floor": floor_s / e2e_s,
                    "d2h_floor": "all ranks copying one slice to pinned host memory at once, nothing else running"},
            # per rank and step: scan, level 1 (which also publishes), pull
            "gpu_launches": 3 * K * world, "clocks": clk_main, "parity": head["parity"],
        }
        if emit:
            print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line if rank == 0 else None


_ORACLE_SCANS = {}


def sharded_parity(replay, table, prio, u_sorted, rank, world, dev, T, rows, L, mode, layout):
    """Parity of one global batch: the indices of every rank's slice against the oracle on all shards'
    priorities, and EVERY gathered byte -- remote requests included -- against read-backs of the
    owner's table: the slices are all-gathered, and every owner compares the requests that landed on
    its shard, wherever they were consumed, with plain cudaMemcpy reads of its own table."""
    import torch
    import torch.distributed as dist
    from gear_b200.sharded import requester_of, route
    n_local = prio.numel()
    Bg = len(u_sorted)
    b = Bg // world
    du = torch.from_numpy(u_sorted).to(dev)
    if mode == "pull":
        colsout, gflat = replay.step_pull(prio, du, layout=layout)
    else:
        colsout, gflat = replay.step_sorted(prio, u_sorted, du, layout=layout)
    torch.cuda.synchronize()
    colsout = [c.contiguous() for c in colsout]
    gflat = gflat.contiguous()
    if world > 1:
        allf = [torch.empty_like(gflat) for _ in range(world)]
        dist.all_gather(allf, gflat)
        allc = []
        for c in colsout:
            parts = [torch.empty_like(c) for _ in range(world)]
            dist.all_gather(parts, c)
            allc.append(parts)
    else:
        allf, allc = [gflat], [[c] for c in colsout]
    flats = [f.cpu().numpy() for f in allf]
    # bytes: every request that landed on MY shard, in whichever rank's slice it sits
    byte_mismatch = checked = remote_checked = 0
    for q in range(world):
        mine = np.nonzero(flats[q] // n_local == rank)[0]
        if len(mine) == 0:
            continue
        host_cols = [allc[c][q].cpu().numpy() for c in range(len(rows))]
        for s in mine:
            fl = int(flats[q][s]) - rank * n_local
            t, ts = divmod(fl, T)
            for c, r in enumerate(rows):
                slot = L * r
                nbytes = min(L, T - ts) * r
                src = t * table.trajectory_stride + table.accu[c] * T + ts * r
                want = table.read(src, nbytes)
                got = host_cols[c][s * slot:(s + 1) * slot]
                byte_mismatch += int((got[:nbytes] != want).sum()) + int(got[nbytes:].any())
            checked += 1
            remote_checked += int(q != rank)
    # indices: every rank's slice against the oracle, shard by shard (rank 0 computes; the
    # priorities do not change during the run, so the oracle's tables are built once)
    key = (prio.data_ptr(), world)
    if key not in _ORACLE_SCANS:
        allp = [torch.empty_like(prio) for _ in range(world)] if world > 1 else [prio]
        if world > 1:
            dist.all_gather(allp, prio)
        _ORACLE_SCANS[key] = None
        if rank == 0:
            from oracle import oracle as O
            _ORACLE_SCANS[key] = [O.scan_mt(p.cpu().numpy(), os.cpu_count() or 1) for p in allp]
        del allp
    mism = torch.tensor([byte_mismatch, checked, remote_checked], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(mism)
    out = None
    if rank == 0:
        # The sharded draw is defined shard by shard: each shard's own cumulative table, shard
        # totals summed in rank order, then the owner-local search.
        from oracle import oracle as O
        scans = _ORACLE_SCANS[key]
        totals = np.array([sc[2] for sc in scans])
        owner, residual, _ = route(totals, u_sorted, world)
        want = np.empty(Bg, np.int64)
        for j in range(world):
            m = owner == j
            want[m] = O.search(scans[j][0], scans[j][1], residual[m]) + j * n_local
        req = requester_of(Bg, world, layout)
        idx_mismatch = sum(int((flats[q] != want[req == q]).sum()) for q in range(world))
        out = {"index_mismatches_vs_oracle": idx_mismatch, "gathered_byte_mismatches": int(mism[0]),
               "requests_byte_checked": int(mism[1]), "remote_requests_byte_checked": int(mism[2]),
               "requests_in_batch": Bg}
    return out
