"""Trajectory-id sharded replay table: global prioritized sampling with one payload exchange.

Sharding follows the reference's loader: the table is cut into blocks of
`capacity_per_rank` trajectories, `owner(g) = g // capacity_per_rank`
(gear/loader/offline_loader.py:131-137), and rank i consumes slice i of the globally
sorted batch (`torch.sort` in gear/sampler/global_sampler.py:131, slices in
offline_loader.py:127-131).  What changes is the traffic:

* the reference gathers candidate indices on dp-rank 0 and broadcasts the sampled ones
  with three point-to-point messages per peer and direction (global_sampler.py:22-56,
  105-152); here every rank already holds the whole batch of variates (they come from a
  counter-based generator or from the caller), the shard totals are all-gathered (8 bytes
  per rank), and every rank derives the complete routing on its own -- no request exchange;
* the reference moves segments with one ncclSend / ncclRecv per segment
  (src/storage/handler.cc:178-191,208-220); here an owner searches and gathers all segments
  asked of it in ONE launch, straight into per-requester regions of a send buffer, and one
  grouped all-to-all per step (`gearb_comm_alltoallv`) lands them in the requester's final
  tensors, which are ordered by owner because the batch is sorted.

`route` and `exchange_plan` are pure host functions (numpy); they are what the CPU-rank
tests exercise.  `ShardedReplay` wires them to the kernels and to NCCL.

A third mode leaves the exchange out altogether (`enable_pull` + `step_pull`): every rank maps
its peers' tables and cumulative-priority tables into its own address space, and the REQUESTER's
kernel routes each request by the all-gathered shard totals (the same arithmetic as `route`),
searches the owner's tables and copies the segment out of the owner's HBM over NVLink, straight
into its final tensors.  The all-gather of the totals is the step's only collective and also its
only synchronisation: with two alternating cumulative tables per rank, a rank cannot start
overwriting a table that a peer may still be reading (the peer's next all-gather contribution
comes after its reads in stream order, and this rank's overwrite comes after that all-gather).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

__all__ = ["route", "exchange_plan", "plan_sorted", "plan_layout", "Plan", "ShardedReplay"]


def route(totals: np.ndarray, u01_sorted: np.ndarray, world: int):
    """Owner and owner-local variate of every request of the global batch.

    totals       float64[world]  total priority of each shard (its l1[-1])
    u01_sorted   float64[B]      the global batch's U[0,1) variates, ascending
    Returns (owner int32[B], residual float64[B], requester int32[B]).
    A request with variate u goes to the shard j with prefix[j] <= u*total < prefix[j+1];
    its residual u*total - prefix[j] is a variate in [0, totals[j]) for the owner's table.
    """
    totals = np.asarray(totals, np.float64)
    u = np.asarray(u01_sorted, np.float64)
    B = len(u)
    if B % world:
        raise ValueError(f"global batch {B} is not a multiple of the world size {world}")
    prefix = np.zeros(world + 1, np.float64)
    acc = 0.0
    for j in range(world):           # in-order float64 sum, like level 1 of the cumulative table
        acc = acc + float(totals[j])
        prefix[j + 1] = acc
    total = prefix[world]
    v = u * total
    v = np.where(v >= 0.0, v, 0.0)
    v = np.where(v < total, v, np.nextafter(total, 0.0))
    owner = np.searchsorted(prefix[1:], v, side="right").astype(np.int32)
    owner = np.minimum(owner, world - 1)
    residual = v - prefix[owner]
    top = np.nextafter(totals[owner], 0.0)
    residual = np.where(residual < totals[owner], residual, top)
    requester = (np.arange(B) // (B // world)).astype(np.int32)
    return owner, residual, requester


def requester_of(B: int, world: int, layout: str = "contiguous") -> np.ndarray:
    """Which rank consumes each position of the sorted global batch: contiguous slices (the
    reference's partition, gear/loader/offline_loader.py:127-131) or dealt round-robin
    ("scattered": rank r takes positions r, r + world, ...; its slice is still ascending, but
    its requests spread over all shards instead of clustering on its own)."""
    if layout == "contiguous":
        return (np.arange(B) // (B // world)).astype(np.int32)
    if layout == "scattered":
        return (np.arange(B) % world).astype(np.int32)
    raise ValueError(f"unknown slice layout {layout!r}")


@dataclass
class Plan:
    """Counts and displacements of one rank, in requests (multiply by a column's slot bytes)."""
    mine: np.ndarray         # positions in the global batch that this rank owns, in batch order
    send_count: np.ndarray   # int64[W]: requests this rank serves for each requester
    send_first: np.ndarray   # int64[W]: first of them inside `mine`
    recv_count: np.ndarray   # int64[W]: requests of this rank's slice served by each owner
    recv_first: np.ndarray   # int64[W]: first slot of them inside the slice (sorted batch => contiguous)
    slice_owner: np.ndarray  # int32[b]: owner of every slot of this rank's slice


def exchange_plan(owner: np.ndarray, requester: np.ndarray, rank: int, world: int) -> Plan:
    """Who sends how much to whom, derived locally from the routing of the whole batch."""
    owner = np.asarray(owner); requester = np.asarray(requester)
    mine = np.nonzero(owner == rank)[0]                      # ascending => grouped by requester
    send_count = np.bincount(requester[mine], minlength=world).astype(np.int64)
    send_first = np.concatenate([[0], np.cumsum(send_count)[:-1]]).astype(np.int64)
    sl = np.nonzero(requester == rank)[0]
    slice_owner = owner[sl].astype(np.int32)
    if len(slice_owner) > 1 and np.any(np.diff(slice_owner) < 0):
        raise ValueError("the batch is not sorted: a rank's slice must be contiguous by owner")
    recv_count = np.bincount(slice_owner, minlength=world).astype(np.int64)
    recv_first = np.concatenate([[0], np.cumsum(recv_count)[:-1]]).astype(np.int64)
    return Plan(mine, send_count, send_first, recv_count, recv_first, slice_owner)


def plan_sorted(totals: np.ndarray, u01_sorted: np.ndarray, rank: int, world: int):
    """The same routing as route() + exchange_plan() for an ASCENDING batch, in O(world log B):
    owners rise with the variate, so the requests a shard owns are one contiguous run of the
    batch.  Returns (plan, total, prefix) where plan.mine is that run as a range."""
    totals = np.asarray(totals, np.float64)
    u = np.asarray(u01_sorted, np.float64)
    B = len(u)
    if B % world:
        raise ValueError(f"global batch {B} is not a multiple of the world size {world}")
    b = B // world
    prefix = np.zeros(world + 1, np.float64)
    acc = 0.0
    for j in range(world):
        acc = acc + float(totals[j])
        prefix[j + 1] = acc
    total = prefix[world]
    v = u * total
    v = np.where(v >= 0.0, v, 0.0)
    v = np.where(v < total, v, np.nextafter(total, 0.0))
    # shard j owns the requests with prefix[j] <= v < prefix[j+1]; the last shard with mass takes the rest
    cut = np.searchsorted(v, prefix[1:world], side="left")
    bounds = np.concatenate([[0], cut, [B]]).astype(np.int64)
    for j in range(world - 1, 0, -1):            # a trailing shard without mass owns nothing
        if totals[j] > 0.0:
            break
        bounds[j] = B
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    slices = np.arange(world + 1, dtype=np.int64) * b

    def overlap(a0, a1, b0, b1):
        return np.maximum(np.minimum(a1, b1) - np.maximum(a0, b0), 0)

    send_count = overlap(lo, hi, slices[:-1], slices[1:]).astype(np.int64)
    send_first = np.concatenate([[0], np.cumsum(send_count)[:-1]]).astype(np.int64)
    recv_count = overlap(bounds[:-1], bounds[1:], slices[rank], slices[rank + 1]).astype(np.int64)
    recv_first = np.concatenate([[0], np.cumsum(recv_count)[:-1]]).astype(np.int64)
    slice_owner = np.repeat(np.arange(world, dtype=np.int32), recv_count)
    return Plan(np.arange(lo, hi), send_count, send_first, recv_count, recv_first, slice_owner), total, prefix


def _owner_bounds(totals: np.ndarray, u01_sorted: np.ndarray, world: int):
    """Cut points of the ascending batch between owners, the global total and the shard prefix."""
    totals = np.asarray(totals, np.float64)
    u = np.asarray(u01_sorted, np.float64)
    B = len(u)
    prefix = np.zeros(world + 1, np.float64)
    acc = 0.0
    for j in range(world):
        acc = acc + float(totals[j])
        prefix[j + 1] = acc
    total = prefix[world]
    v = u * total
    v = np.where(v >= 0.0, v, 0.0)
    v = np.where(v < total, v, np.nextafter(total, 0.0))
    cut = np.searchsorted(v, prefix[1:world], side="left")
    bounds = np.concatenate([[0], cut, [B]]).astype(np.int64)
    for j in range(world - 1, 0, -1):            # a trailing shard without mass owns nothing
        if totals[j] > 0.0:
            break
        bounds[j] = B
    return bounds, total, prefix


def plan_layout(totals: np.ndarray, u01_sorted: np.ndarray, rank: int, world: int, layout: str = "contiguous"):
    """plan_sorted for either slice layout.  Returns (plan, total, prefix, slot_map) where slot_map
    is None (contiguous: an owner's answers are already grouped by requester) or (world, lo, base):
    the owner's request at position q of the batch goes to slot base[q % world] + q // world of its
    send regions, which groups them by requester in the order of the requester's slice."""
    if layout == "contiguous":
        plan, total, prefix = plan_sorted(totals, u01_sorted, rank, world)
        return plan, total, prefix, None
    if layout != "scattered":
        raise ValueError(f"unknown slice layout {layout!r}")
    B = len(u01_sorted)
    if B % world:
        raise ValueError(f"global batch {B} is not a multiple of the world size {world}")
    bounds, total, prefix = _owner_bounds(totals, u01_sorted, world)

    def dealt(a: int, b_: int, q: int):
        """Positions g in [a, b_) with g % world == q: (how many, slot of the first in q's slice)."""
        g0 = a + ((q - a) % world)
        return max(0, -(-(b_ - g0) // world)), g0 // world

    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    send = [dealt(lo, hi, q) for q in range(world)]
    send_count = np.array([c for c, _ in send], np.int64)
    send_first = np.concatenate([[0], np.cumsum(send_count)[:-1]]).astype(np.int64)
    base = np.array([int(send_first[q]) - send[q][1] for q in range(world)], np.int64)
    recv = [dealt(int(bounds[j]), int(bounds[j + 1]), rank) for j in range(world)]
    recv_count = np.array([c for c, _ in recv], np.int64)
    recv_first = np.concatenate([[0], np.cumsum(recv_count)[:-1]]).astype(np.int64)
    slice_owner = np.repeat(np.arange(world, dtype=np.int32), recv_count)
    plan = Plan(np.arange(lo, hi), send_count, send_first, recv_count, recv_first, slice_owner)
    return plan, total, prefix, (world, lo, base)


class ShardedReplay:
    """One rank's shard (table + priorities) plus the exchange.

    table/handler/sampler are gear_b200.core objects of the local shard; `comm` is a
    gear_b200.comm.Communicator (or None when world == 1).  store: the scans keep the level-2
    table (8 bytes of traffic per priority); False: only the partition offsets and block totals
    (4 bytes per priority), and the sampling launches rebuild what each request needs.
    """

    def __init__(self, handler, sampler, columns: Sequence[int], rank: int, world: int, comm=None,
                 max_global_batch: int = 8192, store: bool = True):
        import torch
        from . import _native as N
        self.torch, self.N = torch, N
        self.handler, self.sampler, self.columns = handler, sampler, [int(c) for c in columns]
        self.rank, self.world, self.comm = int(rank), int(world), comm
        self.store = bool(store)
        if world > 1 and comm is None:
            raise ValueError("a communicator is required when world > 1")
        t = handler.table
        self.slots = [handler.patterns[c].length * t.row_bytes[c] for c in self.columns]
        self.n_local = sampler.n
        self.maxB = int(max_global_batch)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        b = self.maxB // world
        self.b_alloc = b
        # One buffer per column: this rank's finished slice (b slots), then what it sends away (worst
        # case: every request of the batch is served by this rank).  An owner's launch writes the
        # requests of its own slice straight into their final slots and the others behind them.
        self._both = [torch.empty((b + self.maxB) * s, dtype=torch.uint8, device=dev) for s in self.slots]
        self._both_flat = torch.empty(b + self.maxB, dtype=torch.int64, device=dev)
        self.recv = [x[: b * s] for x, s in zip(self._both, self.slots)]
        self.send = [x[b * s:] for x, s in zip(self._both, self.slots)]
        self.recv_flat, self.send_flat = self._both_flat[:b], self._both_flat[b:]
        self.totals_dev = torch.empty(world, dtype=torch.float64, device=dev)
        self.totals_host = torch.empty(world, dtype=torch.float64).pin_memory()
        self.res_host = torch.empty(self.maxB, dtype=torch.float64).pin_memory()
        self.res_dev = torch.empty(self.maxB, dtype=torch.float64, device=dev)
        self.last_plan: Optional[Plan] = None
        if comm is not None and world > 1:
            # NCCL sets a pair of ranks up for point-to-point traffic the first time they talk, which
            # takes milliseconds; which pairs a batch needs depends on the draw, so all pairs are
            # connected here instead of inside some later step.
            comm.connect_all()

    # -- step pieces (separate so that a benchmark can time them) ---------------------------
    def scan(self, priorities):
        self.sampler.scan(priorities, store=self.store)

    def gather_totals(self) -> np.ndarray:
        """Shard totals of every rank on the host (one 8-byte-per-rank collective + one sync)."""
        torch = self.torch
        nparts = (self.n_local + self.N.PART - 1) // self.N.PART
        mine = self.sampler.l1[nparts:nparts + 1]
        if self.world == 1:
            self.totals_dev.copy_(mine)
        else:
            self.comm.allgather(mine, self.totals_dev)
        self.totals_host.copy_(self.totals_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.totals_host.numpy().copy()

    def step_sorted(self, priorities, u01_sorted: np.ndarray, u01_sorted_dev, rescan: bool = True,
                    layout: str = "contiguous"):
        """One global batch whose ascending variates are already on the device as well
        (u01_sorted_dev: float64 CUDA tensor with the same values).  The owner reads its run of
        the batch in place and maps it into its own table inside the kernel, so the host only
        does O(world) work per step: one synchronisation for the shard totals (the message sizes of
        the all-to-all depend on them), no other copy in either direction.  layout: how the batch
        is dealt to the ranks (requester_of)."""
        B = len(u01_sorted)
        if B > self.maxB or B % self.world:
            raise ValueError(f"global batch {B}: at most {self.maxB} and a multiple of {self.world}")
        b = B // self.world
        if rescan:
            self.scan(priorities)
        totals = self.gather_totals()
        plan, total, prefix, slot_map = plan_layout(totals, u01_sorted, self.rank, self.world, layout)
        self.last_plan = plan
        m = len(plan.mine)
        if m:
            lo = int(plan.mine[0])
            if self.world > 1:
                # the owner's own requests go straight to their final slots, the others to the send region
                if slot_map is None:
                    slot_map = (-1, lo, [self.rank * b, (self.rank + 1) * b, self.b_alloc])
                else:
                    mod, lo_, base = slot_map
                    base = np.asarray(base, np.int64) + self.b_alloc
                    base[self.rank] = 0
                    slot_map = (mod, lo_, base)
            self.sampler.sample_gather(self.handler, u01_sorted_dev[lo:lo + m], self.columns, self._both, zero_fill=True,
                                       out_flat=self._both_flat, affine=(total, prefix[self.rank]),
                                       flat_offset=self.rank * self.n_local, slot_map=slot_map,
                                       dst_requests=self.b_alloc + m)
        if self.world > 1:
            sc, rc = plan.send_count.copy(), plan.recv_count.copy()
            sc[self.rank] = rc[self.rank] = 0          # already in place
            self.comm.alltoallv(self.send + [self.send_flat], self.recv + [self.recv_flat], self.slots + [8],
                                plan.send_first, sc, plan.recv_first, rc)
        return [r[: b * s] for r, s in zip(self.recv, self.slots)], self.recv_flat[:b]

    def step(self, priorities, u01_sorted: np.ndarray, rescan: bool = True):
        """One global batch, routed request by request on the host (contiguous slices).  Returns
        (column byte tensors of this rank's slice, global step ids)."""
        torch = self.torch
        B = len(u01_sorted)
        if B > self.maxB or B % self.world:
            raise ValueError(f"global batch {B}: at most {self.maxB} and a multiple of {self.world}")
        b = B // self.world
        if rescan:
            self.scan(priorities)
        totals = self.gather_totals()
        owner, residual, requester = route(totals, u01_sorted, self.world)
        plan = exchange_plan(owner, requester, self.rank, self.world)
        self.last_plan = plan
        m = len(plan.mine)

        # owner role: search + gather everything asked of this shard, grouped by requester
        direct = self.world == 1
        dsts = self.recv if direct else self.send
        flat = self.recv_flat if direct else self.send_flat
        if m:
            self.res_host[:m].copy_(torch.from_numpy(residual[plan.mine]))
            self.res_dev[:m].copy_(self.res_host[:m], non_blocking=True)
            self.sampler.sample_gather(self.handler, self.res_dev[:m], self.columns, dsts, scale=False,
                                       zero_fill=True, out_flat=flat)
        if not direct:
            bufs_s = self.send + [self.send_flat]
            bufs_r = self.recv + [self.recv_flat]
            sizes = self.slots + [8]
            self.comm.alltoallv(bufs_s, bufs_r, sizes, plan.send_first, plan.send_count, plan.recv_first,
                                plan.recv_count)
        # global step id = owner * steps_per_shard + owner-local index
        owner_base = torch.from_numpy(plan.slice_owner.astype(np.int64) * self.n_local).to(self.dev)
        return [r[: b * s] for r, s in zip(self.recv, self.slots)], self.recv_flat[:b] + owner_base

    # -- exchange-free mode: requesters read the owners' memory in place ---------------------
    def enable_pull(self, double_buffer: bool = True, ring: bool = False, mailbox: bool = True,
                    priorities=None, copy_l1="auto") -> None:
        """Map every peer's shard into this process (collective: every rank calls it once).

        priorities: a gear_b200.core.DeviceBuffer holding this shard's float32 priorities.  Given,
        the shards keep no level-2 table: every rank scans with the totals-only scan (half the
        traffic), the peers map each other's priorities and block totals, and each rank's level 1
        may travel into the peers' mailboxes with its total (copy_l1), so that a requester searches
        level 1 in its own memory; otherwise it searches the owner's over NVLink.  Either way it
        fetches one 2 KiB block of the owner's priorities per request.  Measured on two GPUs with
        4096 requests per rank: copying costs a step whose requests are nearly all local 14 us
        (181 against 167 us) and saves one with half of them remote 57 us (268 against 325 us), so
        "auto" copies for the scattered layout only.  (A DeviceBuffer because another
        process can only map a whole allocation from its start.)  Needs the mailbox.  While a
        step is in flight anywhere, no rank may change its priorities.

        mailbox: the shard totals travel without a collective -- every rank writes its total and
        the step's number straight into every rank's mailbox, and the pull launch waits (with a
        limit) until all of them have arrived; needs double_buffer.  Otherwise an NCCL all-gather.

        double_buffer (stored tables only): alternate between two cumulative tables so that the
        totals' exchange is the only synchronisation of a step; otherwise one table and a second
        (8-byte) collective closes every step.  ring: stream large requests through bulk-copy
        rings instead of plain 16-byte loads."""
        torch = self.torch
        from . import core
        if self.handler.table.device_ptr == 0:
            raise ValueError("pull mode needs the shards in device memory")
        self._pull_lazy = priorities is not None
        if self._pull_lazy and not (mailbox and double_buffer):
            raise ValueError("pull on tables without level-2 entries needs the mailbox")
        self._pull_ring = bool(ring)
        self._pull_prio = priorities
        self._pull_copy_l1 = copy_l1 if self._pull_lazy else False
        two = double_buffer and not self._pull_lazy
        self._pull_samplers = [self.sampler] + ([core.PrioritySampler(self.n_local)] if two else [])
        self._pull_k = -1
        use_box = mailbox and double_buffer
        self._pull_box = core.DeviceBuffer(core.mailbox_bytes(self.n_local if self._pull_copy_l1 else 0)) if use_box else None
        self._pull_epoch = 0
        own = [self.handler.table.device_ptr] + ([self._pull_box.ptr] if self._pull_box else [])
        if self._pull_lazy:
            b0, b1, _ = self.sampler.block_totals()
            own += [priorities.ptr, b0, b1, *self.sampler.level1_buffers()]
        else:
            for sm in self._pull_samplers:
                own += [sm.cdf_ptr, sm.level1_buffers()[0]]     # these samplers always scan into slot 0
        nh = len(own)
        self._pull_mapped = []
        if self.world == 1:
            ptrs = [own]
        else:
            H = self.N.IPC_HANDLE_BYTES
            mine = b"".join(core.ipc_export(p) for p in own)
            send = torch.frombuffer(bytearray(mine), dtype=torch.uint8).to(self.dev)
            recv = torch.empty(self.world * nh * H, dtype=torch.uint8, device=self.dev)
            self.comm.allgather(send, recv)
            torch.cuda.current_stream().synchronize()
            blob = recv.cpu().numpy().tobytes()
            ptrs = []
            for j in range(self.world):
                if j == self.rank:
                    ptrs.append(own)
                    continue
                row = [core.ipc_open(blob[(j * nh + i) * H:(j * nh + i + 1) * H]) for i in range(nh)]
                self._pull_mapped += row
                ptrs.append(row)
        self._pull_tables = [row[0] for row in ptrs]
        o = 2 if self._pull_box else 1
        self._pull_boxes = [row[1] for row in ptrs] if self._pull_box else None
        if self._pull_lazy:
            self._pull_prios = [row[o] for row in ptrs]
            self._pull_blks = [[row[o + 1] for row in ptrs], [row[o + 2] for row in ptrs]]
            self._pull_l1_remote = [[row[o + 3] for row in ptrs], [row[o + 4] for row in ptrs]]
            self._pull_slot = 0
        else:
            self._pull_cdfs = [[row[o + 2 * k] for row in ptrs] for k in range(len(self._pull_samplers))]
            self._pull_l1s = [[row[o + 1 + 2 * k] for row in ptrs] for k in range(len(self._pull_samplers))]
        self._pull_fence = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self._pull_plans = {}     # prepared pull launches (step_pull)

    def disable_pull(self) -> None:
        """Unmap the peers' memory (collective; call before any rank frees its shard)."""
        from . import core
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.comm.allreduce(self._pull_fence)          # nobody is still reading
            self.torch.cuda.synchronize()
        self._pull_plans = {}
        for p in self._pull_mapped:
            core.ipc_close(p)
        self._pull_mapped = []
        if getattr(self, "_pull_box", None) is not None:
            if self.world > 1:
                self.comm.allreduce(self._pull_fence)      # every rank has unmapped this mailbox
                self.torch.cuda.synchronize()
            self._pull_box.free()
            self._pull_box = None

    def pull_scan(self, priorities, between=None, publish_epoch=None) -> None:
        """Rebuild this shard's cumulative table into the buffer the next step_pull(rescan=False) reads.
        between: called between the scan's two launches (a benchmark records an event there).
        publish_epoch (tables without stored level 2, mailbox, no level-1 copy): the scan's level-1
        launch also writes this shard's total and that epoch into every rank's mailbox."""
        self._pull_k += 1
        sm = self._pull_samplers[self._pull_k % len(self._pull_samplers)]
        if self._pull_lazy:
            # every rank writes the block totals of the step into the same one of its two buffers
            self._pull_slot = (self._pull_epoch + 1) & 1
            sm.select_slot(self._pull_slot)
        store = not self._pull_lazy
        if store:
            sm.select_slot(0)       # the peers hold the address of this sampler's slot-0 tables
        if publish_epoch is not None:
            sm.scan_publish(priorities, self.world, self.rank, self._pull_boxes, publish_epoch)
        elif between is None:
            # with two tables in turn, the launch before this one (the previous pull) reads the other
            sm.scan(priorities, store=store, alternate=store and len(self._pull_samplers) == 2)
        else:
            sm.scan_partitions(priorities, store=store)
            between()
            sm.scan_level1()

    def step_pull(self, priorities, u01_sorted_dev, rescan: bool = True, layout: str = "contiguous", out=None):
        """One global batch without an exchange step: nothing on the host depends on device
        results, so consecutive steps queue back to back on the stream.  u01_sorted_dev: the
        batch's ascending U[0,1) variates as a float64 CUDA tensor (the same on every rank).
        out: (column byte tensors, int64 id tensor) to fill instead of the object's own buffers
        (a caller that keeps several batches in flight passes a different set per batch).
        Returns (column byte tensors of this rank's slice, global step ids)."""
        B = u01_sorted_dev.numel()
        if B > self.maxB or B % self.world:
            raise ValueError(f"global batch {B}: at most {self.maxB} and a multiple of {self.world}")
        b = B // self.world
        nbuf = len(self._pull_samplers)
        copy = (layout == "scattered") if self._pull_copy_l1 == "auto" else bool(self._pull_copy_l1)
        # scan and publish in one call where the publish is only the total and the epoch
        fuse = self._pull_box is not None and self._pull_lazy and not copy
        published = False
        if rescan or self._pull_k < 0:
            self.pull_scan(priorities, publish_epoch=self._pull_epoch + 1 if fuse else None)
            published = fuse
        k = self._pull_k % nbuf
        sm = self._pull_samplers[k]
        if layout == "contiguous":
            first, stride = self.rank * b, 1
        elif layout == "scattered":
            first, stride = self.rank, self.world
        else:
            raise ValueError(f"unknown slice layout {layout!r}")
        recv, recv_flat = (self.recv, self.recv_flat) if out is None else out
        key = None
        if self._pull_box is not None and self._pull_lazy:
            # The pull launch's arguments depend on the slot of the step, the layout, the batch size and the
            # destination buffers only: they are checked and marshalled once per combination, so that the
            # host's share of a step stays well below the GPU's (about 60 us per step otherwise).
            key = (k, self._pull_slot, layout, b, copy, recv[0].data_ptr(), recv_flat.data_ptr())
            hit = self._pull_plans.get(key)
            if hit is not None:
                if (u01_sorted_dev.dtype != self.torch.float64 or not u01_sorted_dev.is_cuda
                        or not u01_sorted_dev.is_contiguous()):
                    raise ValueError("the variates must be a contiguous float64 CUDA tensor")
                self._pull_epoch += 1
                if not published:
                    sm.publish(self.world, self.rank, self._pull_boxes, self._pull_epoch, copy_l1=copy)
                hit[0].run_at(u01_sorted_dev.data_ptr() + 8 * first, self._pull_epoch)
                return hit[1]
        mine = u01_sorted_dev[first:first + b] if stride == 1 else u01_sorted_dev[first:]
        out = [r[: b * s] for r, s in zip(recv, self.slots)], recv_flat[:b]
        common = dict(zero_fill=True, ring=self._pull_ring, out_flat=recv_flat, self_shard=self.rank,
                      count=b, variate_stride=stride)
        if self._pull_box is not None:
            # totals through the mailboxes: no collective, no host involvement
            self._pull_epoch += 1
            e = self._pull_epoch
            if not published:
                sm.publish(self.world, self.rank, self._pull_boxes, e, copy_l1=copy)
            if self._pull_lazy:
                from . import core
                blks = self._pull_blks[self._pull_slot]
                if copy:
                    # level 1 and the block totals of the peers came with their totals: read here, not over NVLink
                    l1s = [sm.l1_ptr if j == self.rank else self._pull_box.ptr + core.mailbox_l1_offset(self.n_local, e, j)
                           for j in range(self.world)]
                    blks = [blks[j] if j == self.rank else self._pull_box.ptr + core.mailbox_blk_offset(self.n_local, e, j)
                            for j in range(self.world)]
                else:
                    l1s = self._pull_l1_remote[self._pull_slot]
                plan = sm.prepare_pull(self.handler, None, None, l1s, self._pull_tables, mine, self.columns, recv,
                                       mailbox=self._pull_box.ptr, prios=self._pull_prios, blks=blks, **common)
                self._pull_plans[key] = (plan, out)
                plan.run(mine, e)
            else:
                sm.pull(self.handler, None, self._pull_cdfs[k], self._pull_l1s[k], self._pull_tables, mine,
                        self.columns, recv, mailbox=self._pull_box.ptr, epoch=e, **common)
            return out
        nparts = (self.n_local + self.N.PART - 1) // self.N.PART
        tot = sm.l1[nparts:nparts + 1]
        if self.world == 1:
            self.totals_dev.copy_(tot)
        else:
            self.comm.allgather(tot, self.totals_dev)   # every shard's scan is complete once this lands
        sm.pull(self.handler, self.totals_dev, self._pull_cdfs[k], self._pull_l1s[k], self._pull_tables, mine,
                self.columns, recv, **common)
        if nbuf == 1 and self.world > 1:
            self.comm.allreduce(self._pull_fence)        # the next scan must not overtake the peers' reads
        return out
