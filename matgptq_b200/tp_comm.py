"""Peer-memory buffers for the row-parallel product fused with its all-reduce (``matgptq_b200_matmul_allreduce``).

In the reference the all-reduce after a row-parallel layer belongs to vLLM (``RowParallelLinear`` reduces what
``MatGPTQLinearMethod.apply`` returns, ``inference_lib/vllm_matgptq.py:180-200``).  Here the product's epilogue
does it: every rank stores its partial sums into every rank's buffer over NVLink and adds what the others
stored.  This module owns the buffers: one symmetric allocation per process group (every rank can address every
rank's copy), a few MB that serve all layers.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _native

class PeerAllReduce:
    """Buffers and handle of one tensor-parallel group.  ``max_rows * max_cols`` bounds ``batch * n_out`` of a call."""

    def __init__(self, group=None, device: torch.device | None = None, max_rows: int = 32, max_cols: int = 8192):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.rank, self.nranks = dist.get_rank(group), dist.get_world_size(group)
        if self.nranks > 8:
            raise ValueError("at most 8 ranks")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.slot_elems = int(max_rows) * int(max_cols)
        data_bytes = 2 * self.nranks * self.slot_elems * 8  # two slot sets of {value, epoch} words per rank
        # plain peer mappings are all the kernel needs; no NVLink multicast object is bound to the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self._buf = symm_mem.empty(data_bytes, dtype=torch.uint8, device=self.device)
        self._buf.zero_()
        self._handle = symm_mem.rendezvous(self._buf, group)
        ptrs = list(self._handle.buffer_ptrs)
        self._ctrl = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.comm = _make_comm(ptrs, self._ctrl.data_ptr(), self.slot_elems, self.rank, self.nranks, push_only=False)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)  # every rank's buffer is zero before anybody stores into it

    def fits(self, batch: int, n_out: int, group_size: int) -> bool:
        return batch < 32 and group_size == 128 and batch * n_out <= self.slot_elems

    def matmul(self, x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, n_out: int, n_in_shard: int,
               bitwidth: int, group_size: int, flags: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """``all_reduce(x_shard @ Wdq_shard.T)`` in one kernel; every rank gets the same bits."""
        return fused_matmul(self.comm, x, packed, scales, n_out, n_in_shard, bitwidth, group_size, flags, out)


def _make_comm(data_ptrs, ctrl_ptr, slot_elems, rank, nranks, push_only) -> _native.Comm:
    comm = _native.Comm()
    for q in range(nranks):
        comm.data[q] = data_ptrs[q]
    comm.ctrl = ctrl_ptr
    comm.slot_elems = slot_elems
    comm.rank, comm.nranks, comm.push_only = rank, nranks, 1 if push_only else 0
    return comm


def fused_matmul(comm: _native.Comm, x, packed, scales, n_out, n_in_shard, bitwidth, group_size, flags, out=None):
    batch = x.size(-2)
    if out is None:
        out = torch.empty((batch, n_out), dtype=x.dtype, device=x.device)
    st = _native.load().matgptq_b200_matmul_allreduce(
        bitwidth, group_size, n_out, n_in_shard, batch, packed.data_ptr(), scales.data_ptr(), x.data_ptr(), out.data_ptr(),
        torch.cuda.current_stream(x.device).cuda_stream, flags, ctypes.byref(comm))
    _native.check(st, "matgptq_b200_matmul_allreduce")
    return out


class LoopbackRanks:
    """All ranks of a group emulated on ONE GPU, for tests: every rank's buffers are local allocations, the ranks'
    products are launched one after the other with ``push_only`` (kernels that wait for each other must not be
    separate launches on one GPU) and ``finish(rank)`` adds up what rank ``rank`` received."""

    def __init__(self, nranks: int, device: torch.device, max_rows: int = 32, max_cols: int = 8192):
        self.nranks, self.slot_elems = nranks, max_rows * max_cols
        self.data = [torch.zeros(2 * nranks * self.slot_elems, dtype=torch.int64, device=device) for _ in range(nranks)]
        self.ctrl = [torch.zeros(4, dtype=torch.int32, device=device) for _ in range(nranks)]
        self.comms = [_make_comm([d.data_ptr() for d in self.data], self.ctrl[r].data_ptr(), self.slot_elems, r, nranks,
                                 push_only=True) for r in range(nranks)]

    def push(self, rank: int, x, packed, scales, n_out, n_in_shard, bitwidth, group_size, flags):
        scratch = torch.empty((x.size(-2), n_out), dtype=x.dtype, device=x.device)  # a push-only launch writes no output
        fused_matmul(self.comms[rank], x, packed, scales, n_out, n_in_shard, bitwidth, group_size, flags, scratch)

    def finish(self, rank: int, batch: int, n_out: int, dtype: torch.dtype, flags: int) -> torch.Tensor:
        out = torch.empty((batch, n_out), dtype=dtype, device=self.data[0].device)
        st = _native.load().matgptq_b200_allreduce_finish(ctypes.byref(self.comms[rank]), out.data_ptr(), n_out, batch,
                                                           torch.cuda.current_stream(out.device).cuda_stream, flags)
        _native.check(st, "matgptq_b200_allreduce_finish")
        return out
