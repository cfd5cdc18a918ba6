"""Batches delivered to pinned host memory with the copy-out of one batch overlapping the
sampling of the next.

The reference's loader hands every batch to the trainer as tensors it gathered on the spot
(`OfflineLoader.fused_iterate`, gear/loader/offline_loader.py:155-204) and a consumer that wants
the batch on the host copies it itself, after the fact.  Over a PCIe link the copy-out of a
batch (config 3: 12.4 MB) takes longer than producing it, so this class keeps `depth` batches
in flight: batch i is sampled and gathered on one stream into buffer i % depth, copied to its
pinned host buffers on a second stream, and handed to the caller when the caller asks for it.

    pipe = HostBatchPipeline(sampler, handler, columns, batch, depth=2)
    pipe.submit(priorities, u01_pinned)        # host variates in; returns at once
    ...
    cols_host, flat_host = pipe.next()         # oldest submitted batch, complete in host memory

The host tensors returned by next() are overwritten by the batch submitted `depth` submits later.
"""
from __future__ import annotations

from collections import deque
from typing import Sequence

import torch

from . import _native as N
from .core import GearError, PrioritySampler, StorageHandler

__all__ = ["HostBatchPipeline"]


class HostBatchPipeline:
    def __init__(self, sampler: PrioritySampler, handler: StorageHandler, columns: Sequence[int], batch: int,
                 depth: int = 2, store_table: bool = False, batch_to_host: bool = True):
        if depth < 1:
            raise GearError(N.ERR_INVALID, "depth must be at least 1")
        self.sampler, self.handler, self.columns = sampler, handler, [int(c) for c in columns]
        self.batch, self.depth, self.store_table = int(batch), int(depth), bool(store_table)
        # batch_to_host=False: the gathered columns stay in device memory for a consumer on the GPU
        # (what the reference's loader returns); only the drawn step ids travel to the host.
        self.batch_to_host = bool(batch_to_host)
        t = handler.table
        self.slots = [handler.patterns[c].length * t.row_bytes[c] for c in self.columns]
        dev = torch.device("cuda", torch.cuda.current_device())
        mk = lambda s: torch.empty(self.batch * s, dtype=torch.uint8, device=dev)
        self._dev_cols = [[mk(s) for s in self.slots] for _ in range(self.depth)]
        self._dev_flat = [torch.empty(self.batch, dtype=torch.int64, device=dev) for _ in range(self.depth)]
        self._dev_u = [torch.empty(self.batch, dtype=torch.float64, device=dev) for _ in range(self.depth)]
        self._host_cols = [[torch.empty(self.batch * s, dtype=torch.uint8).pin_memory() for s in self.slots]
                           for _ in range(self.depth)] if self.batch_to_host else None
        self._host_flat = [torch.empty(self.batch, dtype=torch.int64).pin_memory() for _ in range(self.depth)]
        self._compute = torch.cuda.current_stream()
        self._copy = torch.cuda.Stream()
        self._computed = [torch.cuda.Event() for _ in range(self.depth)]
        self._copied = [torch.cuda.Event() for _ in range(self.depth)]
        self._pending: deque[int] = deque()
        self._submitted = 0

    def submit(self, priorities: torch.Tensor, u01_host: torch.Tensor, rescan: bool = True) -> None:
        """Queue one batch: U[0,1) variates from (pinned) host memory, a scan of `priorities` unless
        rescan is False, then search + gather, then the copy-out.  Returns without waiting."""
        if len(self._pending) == self.depth:
            raise GearError(N.ERR_STATE, "all buffers are in flight: call next() first")
        if u01_host.dtype != torch.float64 or u01_host.numel() != self.batch:
            raise GearError(N.ERR_INVALID, f"variates must be float64 with {self.batch} entries")
        b = self._submitted % self.depth
        cs = self._compute
        cs.wait_event(self._copied[b])            # the buffer's previous copy-out has finished
        with torch.cuda.stream(cs):
            self._dev_u[b].copy_(u01_host, non_blocking=True)
            if rescan:
                self.sampler.scan(priorities, store=self.store_table, stream=cs)
            self.sampler.sample_gather(self.handler, self._dev_u[b], self.columns, self._dev_cols[b], scale=True,
                                       zero_fill=True, out_flat=self._dev_flat[b], stream=cs)
            self._computed[b].record(cs)
        self._copy.wait_event(self._computed[b])
        with torch.cuda.stream(self._copy):
            if self.batch_to_host:
                for h, d in zip(self._host_cols[b], self._dev_cols[b]):
                    h.copy_(d, non_blocking=True)
            self._host_flat[b].copy_(self._dev_flat[b], non_blocking=True)
            self._copied[b].record(self._copy)
        self._pending.append(b)
        self._submitted += 1

    def next(self):
        """The oldest batch in flight, complete: (column byte tensors in pinned host memory -- or, with
        batch_to_host=False, in device memory -- and the flat step ids in pinned host memory)."""
        if not self._pending:
            raise GearError(N.ERR_STATE, "nothing in flight")
        b = self._pending.popleft()
        self._copied[b].synchronize()
        return (self._host_cols[b] if self.batch_to_host else self._dev_cols[b]), self._host_flat[b]

    def drain(self) -> None:
        while self._pending:
            self.next()
