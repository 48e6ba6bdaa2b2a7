"""Communicator classes with the reference's names and call signatures (``MPI_Communicator``,
``NCCL_Communicator``, the ``ncclDataType_t`` / ``ncclRedOp_t`` enums; reference:
``python/athena/communicator/mpi_comm.py:33-85``, ``mpi_nccl_comm.py:47-142``, ``nccl_comm.py:16-89``) on top of
``torch.distributed``: user scripts written against the reference's communicators (``dlarrayNcclAllReduce``,
``dlarrayBroadcast``, ``all_reduce`` of a host array) run unchanged.  The training path does not go through them:
the gradient exchange is ``parallel/fused_allreduce.py`` (one kernel per bucket over NVLink), these classes are the
explicit collectives an example or a test calls by hand (exercised with gloo ranks in
``tests/test_distributed_cpu.py``)."""
from __future__ import annotations

import os
from enum import Enum

import numpy as np
import torch
import torch.distributed as dist

from .. import ndarray
from ..stream import create_stream_handle


class ncclDataType_t(Enum):
    ncclInt8 = 0
    ncclChar = 0
    ncclUint8 = 1
    ncclInt32 = 2
    ncclInt = 2
    ncclUint32 = 3
    ncclInt64 = 4
    ncclUint64 = 5
    ncclFloat16 = 6
    ncclHalf = 6
    ncclFloat32 = 7
    ncclFloat = 7
    ncclFloat64 = 8
    ncclDouble = 8
    ncclNumTypes = 9


class ncclRedOp_t(Enum):
    ncclSum = 0
    ncclProd = 1
    ncclMax = 2
    ncclMin = 3
    ncclNumOps = 4


_REDOP = {ncclRedOp_t.ncclSum: dist.ReduceOp.SUM, ncclRedOp_t.ncclProd: dist.ReduceOp.PRODUCT,
          ncclRedOp_t.ncclMax: dist.ReduceOp.MAX, ncclRedOp_t.ncclMin: dist.ReduceOp.MIN}


def _ensure_group(backend):
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group(backend)


def _flat(arr):
    if isinstance(arr, ndarray.NDArray):
        t = arr.t
        return t.as_strided((t.numel(),), (1,)) if t.is_cuda else t.reshape(-1)
    return torch.from_numpy(arr).reshape(-1)


class MPI_Communicator(object):
    """Host all-reduce (reference ``mpi_comm.py:33-85``), gloo backend."""

    def __init__(self):
        self.comm = None
        self.nRanks, self.myRank = 1, 0

    def MPI_Init(self):
        _ensure_group("gloo")
        self.MPI_GetComm()

    def MPI_GetComm(self):
        self.comm = dist.group.WORLD
        self.myRank, self.nRanks = dist.get_rank(), dist.get_world_size()
        return self.comm

    def MPI_Get_Comm_rank(self):
        return dist.get_rank()

    def MPI_Get_Comm_size(self):
        return dist.get_world_size()

    def rank(self):
        return self.myRank

    def size(self):
        return self.nRanks

    def DLArrayAllReduce(self, dlarray, datatype=ncclDataType_t.ncclFloat32, reduceop=ncclRedOp_t.ncclSum):
        dist.all_reduce(_flat(dlarray), op=_REDOP[reduceop])
        return dlarray

    def allReduce(self, arr):
        return self.DLArrayAllReduce(arr)

    def finish(self):
        if dist.is_initialized():
            dist.destroy_process_group()


def mpi_communicator():
    return MPI_Communicator()


class MPI_NCCL_Communicator(object):
    """One process per GPU (reference ``mpi_nccl_comm.py:47-142``): rank / size /
    local rank discovery, device selection, communicator creation, in-place
    all-reduce of an NDArray followed by a stream sync."""

    def __init__(self):
        self.nRanks, self.myRank, self.localRank = 1, 0, 0
        self.stream = None
        self.ctx = None

    def MPI_Init(self):
        _ensure_group("nccl" if torch.cuda.is_available() else "gloo")

    def MPI_Finalize(self):
        if dist.is_initialized():
            dist.destroy_process_group()

    def MPIGetComm(self):
        return dist.group.WORLD

    def MPI_Comm_rank(self):
        self.myRank = dist.get_rank()
        return self.myRank

    def MPI_Comm_size(self):
        self.nRanks = dist.get_world_size()
        return self.nRanks

    def getLocalRank(self):
        self.localRank = int(os.environ.get("LOCAL_RANK", self.myRank % max(torch.cuda.device_count(), 1)))
        return self.localRank

    def ncclSetDevice(self, device_id):
        if torch.cuda.is_available():
            torch.cuda.set_device(device_id)
        self.ctx = ndarray.gpu(device_id) if torch.cuda.is_available() else ndarray.cpu(0)

    def ncclGetUniqueId(self):
        return None                      # the process group's store distributes the id

    def ncclCommInitRank(self):
        return dist.group.WORLD

    def ncclCommDestroy(self):
        pass

    def streamInit(self):
        self.stream = create_stream_handle(self.ctx) if self.ctx is not None else None

    def dlarrayNcclAllReduce(self, dlarray, datatype=ncclDataType_t.ncclFloat32, reduceop=ncclRedOp_t.ncclSum):
        t = _flat(dlarray)
        if self.stream is not None and self.stream.torch_stream is not None:
            with torch.cuda.stream(self.stream.torch_stream):
                dist.all_reduce(t, op=_REDOP[reduceop])
            self.stream.sync()
        else:
            dist.all_reduce(t, op=_REDOP[reduceop])
        return dlarray

    def ncclAllReduceInit(self):
        self.MPI_Init()
        self.MPI_Comm_rank()
        self.MPI_Comm_size()
        self.getLocalRank()
        self.ncclSetDevice(self.localRank)
        self.ncclGetUniqueId()
        self.ncclCommInitRank()
        self.streamInit()

    def ncclAllReduceFinish(self):
        self.MPI_Finalize()


def mpi_nccl_communicator():
    return MPI_NCCL_Communicator()


class NCCL_Communicator(object):
    """Single process driving several GPUs (reference ``nccl_comm.py:16-89``).
    ``All_Reduce_Ndarray(grads, outs)`` sums one array per device into every
    output array, on per-device streams."""

    def __init__(self, devs, devs_number):
        self.devs = list(devs)[:devs_number]
        self.devs_number = devs_number
        self._create_streams()
        self._init_NCCL()

    def _create_streams(self):
        self.streams = [create_stream_handle(ndarray.gpu(d)) for d in self.devs] if torch.cuda.is_available() \
            else [None] * self.devs_number

    def _destroy_streams(self):
        self.streams = []

    def _init_NCCL(self):
        self.ready = True

    def _destroy_NCCL_comms(self):
        self.ready = False

    def _stream_sync(self):
        for s in self.streams:
            if s is not None:
                s.sync()

    def show_property(self):
        print("devices:", self.devs, "number:", self.devs_number)

    def All_Reduce_Ndarray(self, gradient_list, allreduced_gradient_list):
        assert len(gradient_list) == self.devs_number == len(allreduced_gradient_list)
        if torch.cuda.is_available() and all(g.t.is_cuda for g in gradient_list):
            outs = [o.t for o in allreduced_gradient_list]
            for o, g in zip(outs, gradient_list):
                o.copy_(g.t)
            torch.cuda.nccl.all_reduce(outs)
        else:
            total = sum(g.t.cpu() for g in gradient_list)
            for o in allreduced_gradient_list:
                o.t.copy_(total)
        self._stream_sync()

    all_reduce = All_Reduce_Ndarray


def nccl_communicator(devs, devs_number):
    return NCCL_Communicator(devs, devs_number)
