"""Online ingestion: simulators fill trajectories while the trainer samples them.

`IndexServer` / `IndexClient` wrap the C ABI's gearb_ingest_* (the reference's
SharedMemoryIndexServer / SharedMemoryIndexClient, src/index/server.cc, src/index/client.cc).
`OnlineIngest` is what the reference leaves to its callers: one trainer-side step that scans the
simulators' slots, writes what they committed into the host-side weight / length arrays AND into
the device-side cumulative-priority table with the incremental update (gearb_sampler_update:
only the partitions of the touched trajectories are rescanned), and hands the inference
requests back to whoever answers them.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _native as N
from ._native import GearError, call, lib

__all__ = ["IndexServer", "IndexClient", "OnlineIngest"]


class IndexServer:
    """Trainer side.  One instance per shard: `capacity` trajectories starting at `index_offset`."""

    def __init__(self, key: int, num_clients: int, index_offset: int, capacity: int):
        self.key, self.num_clients = int(key), int(num_clients)
        self.index_offset, self.capacity = int(index_offset), int(capacity)
        self._h = C.c_void_p(0)
        call("gearb_ingest_server_create", self.key, self.num_clients, self.index_offset, self.capacity,
             C.byref(self._h))
        m = self.num_clients
        self.infer_src = np.zeros(m, np.int32)
        self.infer_idx = np.zeros(m, np.int64)
        self.infer_ts = np.zeros(m, np.int64)
        self.upd_idx = np.zeros(2 * m, np.int64)
        self.upd_ts = np.zeros(2 * m, np.int64)
        self.upd_w = np.zeros(2 * m, np.float32)

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(C.c_void_p)

    def scan(self):
        """One pass over the slots.  Returns (n_infer, n_updates); the arrays infer_* / upd_* hold them."""
        ni, nu = C.c_int64(0), C.c_int64(0)
        call("gearb_ingest_server_scan", self._h, self._p(self.infer_src), self._p(self.infer_idx),
             self._p(self.infer_ts), self.num_clients, C.byref(ni), self._p(self.upd_idx), self._p(self.upd_ts),
             self._p(self.upd_w), 2 * self.num_clients, C.byref(nu))
        return ni.value, nu.value

    def update(self, n: int) -> None:
        """The first n recorded updates into the weight / length arrays."""
        call("gearb_ingest_server_update", self._h, self._p(self.upd_idx), self._p(self.upd_ts), self._p(self.upd_w),
             int(n))

    def callback(self, srcs: np.ndarray) -> None:
        srcs = np.ascontiguousarray(srcs, np.int32)
        call("gearb_ingest_server_callback", self._h, self._p(srcs), len(srcs))

    @property
    def weights(self) -> np.ndarray:
        p = lib.gearb_ingest_server_weights(self._h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(self.capacity,))

    @property
    def timesteps(self) -> np.ndarray:
        p = lib.gearb_ingest_server_timesteps(self._h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int64)), shape=(self.capacity,))

    @property
    def free_count(self) -> int:
        return int(lib.gearb_ingest_server_free_count(self._h))

    def get_state(self) -> bytes:
        n = lib.gearb_ingest_server_get_state(self._h, None, 0)
        buf = C.create_string_buffer(n)
        if lib.gearb_ingest_server_get_state(self._h, buf, n) != n:
            raise GearError(N.ERR_STATE, "ingest server: state changed size while it was read")
        return buf.raw

    def set_state(self, state: bytes) -> None:
        call("gearb_ingest_server_set_state", self._h, C.create_string_buffer(bytes(state), len(state)), len(state))
        self.index_offset = int(np.frombuffer(state[:48], np.int64)[2])     # the image carries its shard's offset

    def close(self) -> None:
        if self._h:
            lib.gearb_ingest_server_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class IndexClient:
    """Simulator side: slot `rank` of the server's segment."""

    def __init__(self, key: int, rank: int, num_clients: int):
        self.key, self.rank, self.num_clients = int(key), int(rank), int(num_clients)
        self._h = C.c_void_p(0)

    def connect(self) -> int:
        """0 once attached, -1 while the server's segment does not exist (callers retry, as with
        the reference's connect(), src/index/client.cc:19-27)."""
        if self._h:
            return 0
        try:
            call("gearb_ingest_client_create", self.key, self.rank, self.num_clients, C.byref(self._h))
        except GearError as e:
            if e.code == N.ERR_STATE:
                return -1
            raise
        return 0

    def acquire(self, timeout_ms: int = 10_000) -> int:
        """Blocks (up to the limit) until this simulator holds a trajectory; returns its index."""
        t = C.c_int64(0)
        call("gearb_ingest_client_acquire", self._h, int(timeout_ms), C.byref(t))
        return t.value

    def wait(self, timeout_ms: int = 10_000) -> None:
        call("gearb_ingest_client_wait", self._h, int(timeout_ms))

    def release(self) -> None:
        call("gearb_ingest_client_release", self._h)

    def step_inc(self) -> int:
        return int(lib.gearb_ingest_client_step(self._h))

    def writeback(self, terminated: bool, alloc_new: bool, weight: float = 0.0) -> int:
        return int(lib.gearb_ingest_client_writeback(self._h, int(bool(terminated)), int(bool(alloc_new)), float(weight)))

    def status(self) -> dict:
        out = (C.c_int64 * 7)()
        w = C.c_double(0.0)
        call("gearb_ingest_client_status", self._h, out, C.byref(w))
        keys = ("ownership", "terminated", "alloc", "valid", "tindex", "timestep", "on_the_fly")
        d = dict(zip(keys, [int(x) for x in out]))
        d["weight"] = w.value
        return d

    def get_index(self) -> int:
        return self.status()["tindex"]

    def get_timestep(self) -> int:
        return self.status()["timestep"]

    def close(self) -> None:
        if self._h:
            lib.gearb_ingest_client_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class OnlineIngest:
    """Trainer-side step of the online path.

    server: IndexServer of this shard.  sampler / priorities: a gear_b200.core.PrioritySampler
    over one float32 priority per trajectory of the shard and the CUDA tensor it was scanned from
    (optional: without them only the host arrays are kept).  After every `step()` the device
    table equals a full scan of the server's weights, bit for bit.  table: a
    gear_b200.core.TrajectoryTable with a shared-memory host copy, which the simulators write,
    and an uploaded device copy: every committed trajectory's bytes are copied to the device
    copy before its weight makes it selectable (same stream, so the order holds on the device)."""

    def __init__(self, server: IndexServer, sampler=None, priorities=None, table=None):
        self.server, self.sampler, self.priorities, self.table = server, sampler, priorities, table
        if sampler is not None:
            import torch
            if priorities is None or priorities.numel() != server.capacity or sampler.n != server.capacity:
                raise GearError(N.ERR_INVALID, "one priority per trajectory of the shard is required")
            self._torch = torch
            m = 2 * server.num_clients
            self._idx_host = torch.empty(m, dtype=torch.int64).pin_memory()
            self._w_host = torch.empty(m, dtype=torch.float32).pin_memory()
            self._idx_dev = torch.empty(m, dtype=torch.int64, device=priorities.device)
            self._w_dev = torch.empty(m, dtype=torch.float32, device=priorities.device)

    def step(self):
        """Scan, apply, and return the inference requests as (slots, trajectories, timesteps) copies.
        The caller answers them and hands the slots back with server.callback(slots)."""
        s = self.server
        ni, nu = s.scan()
        if nu:
            s.update(nu)
            if self.table is not None:
                stride = self.table.trajectory_stride
                for k in range(nu):
                    if s.upd_w[k] > 0.0:          # a finished trajectory (allocations come with weight 0)
                        self.table.upload_range((int(s.upd_idx[k]) - s.index_offset) * stride, stride)
            if self.sampler is not None:
                torch = self._torch
                self._idx_host[:nu] = torch.from_numpy(s.upd_idx[:nu] - s.index_offset)
                self._w_host[:nu] = torch.from_numpy(s.upd_w[:nu])
                self._idx_dev[:nu].copy_(self._idx_host[:nu], non_blocking=True)
                self._w_dev[:nu].copy_(self._w_host[:nu], non_blocking=True)
                self.sampler.update(self.priorities, self._idx_dev[:nu], self._w_dev[:nu])
                torch.cuda.current_stream().synchronize()     # the pinned staging arrays are reused next step
        return s.infer_src[:ni].copy(), s.infer_idx[:ni].copy(), s.infer_ts[:ni].copy()
