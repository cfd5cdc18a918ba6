"""NCCL communicator over the C ABI (gearb_comm_*), the counterpart of the reference's
NcclCommunicator (src/nccl_comm.cc) and its Python wrapper (gear/comm/nccl.py).

The reference exchanges the 128-byte unique id over a TCP socket (gear/comm/nccl.py:14-38);
here it travels through whatever the launcher already provides: `from_torch_distributed`
broadcasts it over an initialised torch.distributed group.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np
import torch

from . import _native as N
from ._native import call, lib


def create_nccl_id() -> bytes:
    """comm.create_nccl_id (src/nccl_comm.cc:4-10)."""
    buf = C.create_string_buffer(128)
    call("gearb_comm_unique_id", buf)
    return buf.raw


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Communicator:
    def __init__(self, rank: int, world: int, nccl_id: bytes):
        if len(nccl_id) != 128:
            raise N.GearError(N.ERR_INVALID, "the NCCL id must be 128 bytes")
        self._h = C.c_void_p(0)
        self.rank_, self.world = int(rank), int(world)
        call("gearb_comm_create", self.rank_, self.world, nccl_id, C.byref(self._h))

    @staticmethod
    def from_torch_distributed(group=None) -> "Communicator":
        """One communicator per process; the id is broadcast from rank 0 of the group."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [create_nccl_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return Communicator(rank, world, box[0])

    # names of the reference's binding (src/nccl_comm.cc:103-113)
    def rank(self) -> int:
        return self.rank_

    def size(self) -> int:
        return self.world

    def device(self) -> int:
        d = C.c_int(0)
        call("gearb_comm_info", self._h, None, None, C.byref(d))
        return d.value

    def send(self, t: torch.Tensor, dst: int) -> None:
        call("gearb_comm_send", self._h, C.c_void_p(t.data_ptr()), t.numel() * t.element_size(), int(dst), _stream())

    def recv(self, t: torch.Tensor, src: int) -> None:
        call("gearb_comm_recv", self._h, C.c_void_p(t.data_ptr()), t.numel() * t.element_size(), int(src), _stream())

    def allreduce(self, t: torch.Tensor) -> None:
        dt = {torch.float32: N.DT_F32, torch.float64: N.DT_F64, torch.int64: N.DT_I64, torch.float16: N.DT_F16}.get(t.dtype)
        if dt is None:
            raise N.GearError(N.ERR_INVALID, f"allreduce: unsupported dtype {t.dtype}")
        call("gearb_comm_allreduce_sum", self._h, C.c_void_p(t.data_ptr()), t.numel(), dt, _stream())

    def allgather(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        nbytes = send.numel() * send.element_size()
        if recv.numel() * recv.element_size() < nbytes * self.world:
            raise N.GearError(N.ERR_INVALID, "allgather: receive buffer too small")
        call("gearb_comm_allgather", self._h, C.c_void_p(send.data_ptr()), C.c_void_p(recv.data_ptr()), nbytes, _stream())

    def alltoallv(self, send: Sequence[torch.Tensor], recv: Sequence[torch.Tensor], unit_bytes: Sequence[int],
                  send_first, send_count, recv_first, recv_count) -> None:
        """Variable all-to-all over several buffer pairs at once.  Counts and displacements are in
        requests and shared by all pairs; pair k moves unit_bytes[k] bytes per request."""
        nb, W = len(send), self.world
        so = np.empty(nb * W, np.int64); sb = np.empty_like(so); ro = np.empty_like(so); rb = np.empty_like(so)
        for k, u in enumerate(unit_bytes):
            so[k * W:(k + 1) * W] = np.asarray(send_first, np.int64) * u
            sb[k * W:(k + 1) * W] = np.asarray(send_count, np.int64) * u
            ro[k * W:(k + 1) * W] = np.asarray(recv_first, np.int64) * u
            rb[k * W:(k + 1) * W] = np.asarray(recv_count, np.int64) * u
        p = lambda a: a.ctypes.data_as(C.POINTER(C.c_int64))
        call("gearb_comm_alltoallv", self._h, nb, (C.c_void_p * nb)(*[t.data_ptr() for t in send]), p(so), p(sb),
             (C.c_void_p * nb)(*[t.data_ptr() for t in recv]), p(ro), p(rb), _stream())

    def connect_all(self) -> None:
        """One small message between every pair of ranks (collective).  NCCL builds the connection
        of a pair on its first send/recv, which takes milliseconds; after this call no later
        all-to-all pays for that, whichever pairs it happens to use."""
        W = self.world
        if W <= 1:
            return
        s = torch.zeros(W * 16, dtype=torch.uint8, device="cuda")
        r = torch.empty(W * 16, dtype=torch.uint8, device="cuda")
        ones = np.ones(W, np.int64)
        first = np.arange(W, dtype=np.int64)
        for _ in range(2):
            self.alltoallv([s], [r], [16], first, ones, first, ones)
        torch.cuda.current_stream().synchronize()

    def close(self) -> None:
        if self._h:
            lib.gearb_comm_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
