"""Communicator classes with the reference's method names
(``python/athena/communicator/{mpi_comm,mpi_nccl_comm,nccl_comm}.py``), carried by
``torch.distributed`` (NCCL on GPUs, gloo on hosts) instead of MPI / raw NCCL
handles; rendezvous comes from the usual ``RANK`` / ``WORLD_SIZE`` /
``MASTER_ADDR`` / ``MASTER_PORT`` environment (``torchrun`` replaces ``mpirun``)."""
from .comms import (MPI_Communicator, mpi_communicator, MPI_NCCL_Communicator, mpi_nccl_communicator,
                    NCCL_Communicator, nccl_communicator, ncclDataType_t, ncclRedOp_t)

__all__ = ["MPI_Communicator", "mpi_communicator", "MPI_NCCL_Communicator", "mpi_nccl_communicator",
           "NCCL_Communicator", "nccl_communicator", "ncclDataType_t", "ncclRedOp_t"]
