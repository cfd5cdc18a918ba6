"""gear/comm: the NCCL wrapper.  (The reference's wrappers call `lgcm.NcclComm`, a name its
module never registers -- src/nccl_comm.cc:105 registers NcclCommunicator.)"""
from ...libgear.comm import NcclCommunicator, create_nccl_id  # noqa: F401

__all__ = ["NcclCommunicator", "create_nccl_id"]
