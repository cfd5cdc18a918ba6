"""`libgear.comm` (src/nccl_comm.cc:103-113): create_nccl_id and NcclCommunicator."""
from __future__ import annotations

from ..comm import Communicator, create_nccl_id  # noqa: F401


class NcclCommunicator(Communicator):
    """NcclCommunicator(rank, ws, id) with rank()/size()/device()/send/recv/allreduce."""

    def __init__(self, rank: int, ws: int, id: bytes):  # noqa: A002  (the reference's argument name)
        super().__init__(rank, ws, bytes(id))


__all__ = ["create_nccl_id", "NcclCommunicator"]
