"""Symmetric-memory buffers and the fused all-reduce + add + RMSNorm call of the tensor-parallel decode step.

Every rank allocates the same block with torch's symmetric-memory allocator and exchanges the mappings once
(`rendezvous`); afterwards each rank holds plain device pointers to all peers' blocks.  The row-parallel linears
write their partial outputs straight into the local block; `sbvr_allreduce_add_rmsnorm_f16` then reads all peers'
partials over NVLink (ordinary loads) and finishes the layer's residual add and RMSNorm in the same launch.
"""
from __future__ import annotations

import torch

from sbvr import _lib


class SymmetricAllReduce:
    FLAG_BYTES = 1024

    def __init__(self, group, device, max_rows: int, hidden: int, calls_per_step: int):
        import os
        import torch.distributed as dist
        # the all-reduce kernel reads the peers with plain loads: the allocator need not (and, so that a rank that dies
        # does not leave peers bound to an NVLink multicast object, should not) create a multicast mapping
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_rows, self.hidden, self.calls_per_step = max_rows, hidden, calls_per_step
        self.buf_elems = max_rows * hidden
        data_bytes = 2 * self.buf_elems * 2
        self.block = symm.empty(data_bytes + self.FLAG_BYTES, dtype=torch.uint8, device=device)
        self.block.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.block, group)
        self.handle.barrier()                       # every rank's flags are zero before anyone signals
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.bufs_dev = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.flags_dev = torch.tensor([p + data_bytes for p in ptrs], dtype=torch.int64, device=device)
        self.step = torch.zeros(1, dtype=torch.int32, device=device)
        self.local = self.block[:data_bytes].view(torch.float16).view(2, max_rows, hidden)

    def partial_out(self, call_idx: int, rows: int) -> torch.Tensor:
        """Where the row-parallel linear of call `call_idx` of this step writes its [rows, hidden] partial."""
        return self.local[call_idx & 1, :rows]

    def reduce_add_rmsnorm(self, call_idx: int, h: torch.Tensor, weight: torch.Tensor, y: torch.Tensor, rows: int,
                           eps: float, ws, stream: int):
        _lib.check(_lib.lib.sbvr_allreduce_add_rmsnorm_f16(
            self.bufs_dev.data_ptr(), self.flags_dev.data_ptr(), self.step.data_ptr(), self.calls_per_step, call_idx,
            self.rank, self.world, self.buf_elems, h.data_ptr(), weight.data_ptr(), h.data_ptr(), y.data_ptr(), rows,
            self.hidden, eps, ws.handle, stream), "sbvr_allreduce_add_rmsnorm_f16")

    def end_step(self):
        self.step.add_(1)
