"""gear/loader/offline_loader.py: OfflineLoader with the reference's constructor, method names
and return shapes (:39-357).

`next(loader)` = `fused_iterate()` returns `(timesteps, [one tensor per subscribed column])`,
each tensor `[batch, pattern.length, *column_shape]` in the column's dtype, zero padded.

What differs from the reference underneath:
* all subscribed columns are gathered by ONE launch (the reference launches once per column
  after a `torch.zeros` each, :178-203);
* the trajectory lengths of a batch are looked up on the device (the reference indexes a host
  tensor with `.cpu()` per peer, :168-177);
* with more than one data-parallel rank every rank receives its slice of the sorted batch
  through one grouped all-to-all (the reference's multi-rank branch never advances its slot
  pointer, :191-202, and only fills slot 0).
"""
import logging
import pathlib
from typing import Any, Dict, List, Literal, Sequence, Union

import numpy as np
import torch

from ...libgear import core as glibc
from ...sharded import exchange_plan
from ..dataset import SharedDataset
from ..dtypes import CVT_DTYPES_GEAR_TO_TORCH
from ..sampler import TopKSampler, UniformSampler, WeightedSampler
from ..utils import get_local_node_hashed_int32
from .basic_loader import BasicLoader

_SAMPLERS = {"Uniform": UniformSampler, "Weighted": WeightedSampler, "Topk": TopKSampler, "TopK": TopKSampler}


def ensure_dataset(dataset):
    if isinstance(dataset, SharedDataset):
        return dataset
    if isinstance(dataset, (str, pathlib.Path)):
        return SharedDataset().load(dataset)
    raise NotImplementedError(f"Conversion from {dataset} to SharedDataset is unknown")


class OfflineLoader(BasicLoader):
    @staticmethod
    def create(data_path, batch_size: int, mpu, sampling_method: Literal["Uniform", "Weighted", "Topk"] = "Uniform",
               patterns=None, key: Union[int, None] = None, attach: bool = True):
        if key is None:
            key = get_local_node_hashed_int32()
        dataset = SharedDataset().load(data_path, key)
        return OfflineLoader(dataset, batch_size, mpu, sampling_method, patterns)

    def __init__(self, dataset, batch_size: int, mpu, sampling_method="Uniform",
                 patterns: List[Union[Dict[str, Any], glibc.SubscribePattern]] = None, logger: logging.Logger = None):
        super().__init__(batch_size)
        self._dataset = ensure_dataset(dataset)
        self._handler, self._table, self._iset = self._dataset._handler, self._dataset._table, self._dataset._iset
        spec = self._table.get_table_spec()
        self._sub_cols = [spec.index(p["name"]) for p in patterns]
        if any(c < 0 for c in self._sub_cols):
            raise RuntimeError("OfflineLoader: a pattern names a column the table does not have")
        self._patterns = [
            glibc.SubscribePattern(p["offset"], p["length"],
                                   glibc.SubscribePattern.PadOption.tail if p.get("pad", "tail") == "tail"
                                   else glibc.SubscribePattern.PadOption.head)
            for p in patterns
        ]
        self._handler.set(self._sub_cols, self._patterns)
        self._mpu = mpu
        self._dp_rank = mpu.get_data_parallel_rank()
        self._dp_world = mpu.get_data_parallel_world_size()
        self._dp_capacity = self._iset.local_capacity
        self._batch_size = batch_size
        self._logger = logger if logger else logging.Logger(name="OfflineLoader", level=logging.DEBUG)
        self._sampler = _SAMPLERS[sampling_method](mpu, seed=42)
        self._indices = torch.arange(self._iset.local_capacity, dtype=torch.long, device=mpu.device) + self._iset.index_offset
        self._device_timesteps = None
        self._comm = None

    @property
    def table_spec(self):
        return self._table.get_table_spec() if self._table else None

    # -- the reference's helpers -----------------------------------------------------------
    def partition_indices(self, global_indices):
        """parts[i][j]: indices of rank i's slice that rank j owns (:123-140)."""
        batch = global_indices.size(0)
        slice_size = max(int(batch / self._dp_world), 1)
        parts = [[None] * self._dp_world for _ in range(self._dp_world)]
        for i in range(self._dp_world):
            assigned = global_indices[slice_size * i: slice_size * (i + 1)]
            for j in range(self._dp_world):
                lo = j * self._dp_capacity
                parts[i][j] = assigned[(lo <= assigned) & (assigned < lo + self._dp_capacity)]
        return parts

    def generate_rank_comm_order(self):
        """Rotation that starts at (W - rank) % W (:142-153)."""
        ranks = [(0 - self._dp_rank + self._dp_world) % self._dp_world]
        for i in range(1, self._dp_world):
            ranks.append((ranks[i - 1] + 1) % self._dp_world)
        return ranks

    # -- batches ---------------------------------------------------------------------------
    def _timesteps_dev(self):
        # trajectory lengths change only when the dataset is written; refresh per batch is cheap
        t = self._iset.timesteps
        if self._device_timesteps is None or self._device_timesteps.numel() != t.numel():
            self._device_timesteps = torch.empty(t.numel(), dtype=torch.long, device=self._mpu.device)
        self._device_timesteps.copy_(t, non_blocking=True)
        return self._device_timesteps

    def _alloc(self, n):
        out = []
        for i, col_id in enumerate(self._sub_cols):
            cspec = self._table.get_column_spec(col_id)
            out.append(torch.empty((n, self._patterns[i].length) + tuple(cspec.shape),
                                   dtype=CVT_DTYPES_GEAR_TO_TORCH[cspec.dtype], device=self._mpu.device))
        return out

    def _gather_local(self, local_idx, dsts):
        tss = self._timesteps_dev()[local_idx]
        self._handler.gather(self._sub_cols, local_idx.contiguous(), tss, tss, dsts, zero_fill=True)
        return tss

    def fused_iterate(self):
        sampled = self._sampler.sync_sample(self._indices, self._iset.weights, self._batch_size * self._dp_world)
        if self._dp_world == 1:
            data = self._alloc(self._batch_size)
            tss = self._gather_local(sampled - self._iset.index_offset, data)
            return tss, data
        return self._exchange(sampled)

    def _exchange(self, sampled):
        """Every rank serves the requests it owns and receives its slice, one all-to-all."""
        from ...comm import Communicator
        if self._comm is None:
            self._comm = Communicator.from_torch_distributed(self._mpu.get_data_parallel_group())
        W, b = self._dp_world, self._batch_size
        g = sampled.cpu().numpy()
        owner = (g // self._dp_capacity).astype(np.int32)
        requester = (np.arange(len(g)) // b).astype(np.int32)
        plan = exchange_plan(owner, requester, self._dp_rank, W)
        m = len(plan.mine)
        send = self._alloc(max(m, 1))
        send_ts = torch.zeros(max(m, 1), dtype=torch.long, device=self._mpu.device)
        if m:
            local = torch.from_numpy(g[plan.mine] % self._dp_capacity).to(self._mpu.device)
            send_ts[:m] = self._gather_local(local, [s[:m] for s in send])
        recv = self._alloc(b)
        recv_ts = torch.zeros(b, dtype=torch.long, device=self._mpu.device)
        units = [r[0].numel() * r.element_size() for r in recv] + [8]
        self._comm.alltoallv([s.view(-1).view(torch.uint8) for s in send] + [send_ts.view(torch.uint8)],
                             [r.view(-1).view(torch.uint8) for r in recv] + [recv_ts.view(torch.uint8)],
                             units, plan.send_first, plan.send_count, plan.recv_first, plan.recv_count)
        return recv_ts, recv

    def low_level_controlled_iterate(self):
        """The two-step route of the reference: host-side `sub` then `vcopy` (:206-278)."""
        sampled = self._sampler.sync_sample(self._indices, self._iset.weights, self._batch_size * self._dp_world).cpu()
        if self._dp_world != 1:
            raise NotImplementedError("the two-step route serves a single data-parallel rank; use fused_iterate")
        return self.exposed_low_level_controlled_iterate(sampled)

    def __next__(self):
        return self.fused_iterate()

    def exposed_fused_iterate(self, indices):
        """Gather the given (local) trajectory indices (:284-309)."""
        idx = torch.as_tensor(indices, dtype=torch.long).to(self._mpu.device)
        data = self._alloc(idx.numel())
        self._gather_local(idx % self._dp_capacity, data)
        return data

    def exposed_low_level_controlled_iterate(self, indices):
        indices = torch.as_tensor(indices, dtype=torch.long).cpu()
        n = indices.numel()
        src_offsets = torch.zeros(n, dtype=torch.long)
        dst_offsets = torch.zeros(n, dtype=torch.long)
        copied_lens = torch.zeros(n, dtype=torch.long)
        tss = self._iset.timesteps[indices % self._dp_capacity]
        data = []
        for i, col_id in enumerate(self._sub_cols):
            cspec = self._table.get_column_spec(col_id)
            out = torch.zeros((n, self._patterns[i].length) + tuple(cspec.shape),
                              dtype=CVT_DTYPES_GEAR_TO_TORCH[cspec.dtype], device=self._mpu.device)
            max_len = self._handler.sub(glibc.Int64Span.from_tensor(indices), glibc.Int64Span.from_tensor(tss),
                                        glibc.Int64Span.from_tensor(tss), col_id,
                                        glibc.Int64Span.from_tensor(src_offsets), glibc.Int64Span.from_tensor(dst_offsets),
                                        glibc.Int64Span.from_tensor(copied_lens))
            glibc.vcopy(self._table.get_address(), out, src_offsets.cuda(), dst_offsets.cuda(), copied_lens.cuda(), max_len)
            data.append(out)
        torch.cuda.synchronize()
        return tss, data
