"""Symmetric-memory buffers and the fused all-reduce + add + RMSNorm calls of the tensor-parallel decode step.

Every rank allocates the same block with torch's symmetric-memory allocator and exchanges the mappings once
(`rendezvous`); afterwards each rank holds plain device pointers to all peers' blocks.  Two forms:

* up to four rows (decode): the row-parallel linear's own epilogue stores its result as epoch-tagged 8-byte packets into
  every rank's receive area (`sbvr_linear_push_f16`), and `sbvr_ll_reduce_add_rmsnorm_f16` adds the packets that have
  arrived in the local area and finishes the residual add and RMSNorm: one NVLink crossing, no flags;
* more rows: the linears write their partial outputs into the local block and `sbvr_allreduce_add_rmsnorm_f16` reads all
  peers' partials over NVLink (ordinary loads) after a flag exchange.
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
        self.push_rows = min(4, max_rows)           # the pushed form exists for the decode GEMV (up to four rows)
        recv_off = data_bytes + self.FLAG_BYTES
        recv_bytes = 2 * self.world * self.push_rows * (hidden // 2) * 8
        self.block = symm.empty(recv_off + recv_bytes, dtype=torch.uint8, device=device)
        self.block.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.block, group)
        self.handle.barrier()                       # every rank's flags are zero before anyone signals
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.bufs_dev = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.flags_dev = torch.tensor([p + data_bytes for p in ptrs], dtype=torch.int64, device=device)
        self.recv_local = ptrs[self.rank] + recv_off
        self.step = torch.zeros(1, dtype=torch.int32, device=device)
        # one push descriptor per call of a step, in device memory (sbvr_push_desc_t)
        import ctypes
        descs = (_lib.PushDesc * calls_per_step)()
        for c in range(calls_per_step):
            for r, p in enumerate(ptrs):
                descs[c].peer_recv[r] = p + recv_off
            descs[c].step = self.step.data_ptr()
            descs[c].calls_per_step, descs[c].call_idx = calls_per_step, c
            descs[c].rank, descs[c].world, descs[c].rows_max = self.rank, self.world, self.push_rows
        raw = torch.frombuffer(bytearray(bytes(descs)), dtype=torch.uint8)
        self.push_descs = raw.to(device)
        self.push_desc_bytes = ctypes.sizeof(_lib.PushDesc)
        self.local = self.block[:data_bytes].view(torch.float16).view(2, max_rows, hidden)

    def partial_out(self, call_idx: int, rows: int) -> torch.Tensor:
        """Where the row-parallel linear of call `call_idx` of this step writes its [rows, hidden] partial."""
        return self.local[call_idx & 1, :rows]

    def emits_digits(self, rows: int) -> bool:
        """Whether the reduce kernels can leave their result as activation digits for a decode GEMV that would otherwise
        launch a quantiser kernel of its own (rows longer than 4096 elements, up to four of them)."""
        return rows <= 4 and self.hidden % 2048 == 0 and rows * (self.hidden // 256) > 16

    def reduce_add_rmsnorm(self, call_idx: int, h: torch.Tensor, weight: torch.Tensor, y: torch.Tensor, rows: int,
                           eps: float, ws, stream: int, emit_digits: bool = False) -> bool:
        """Returns whether the digits were written (emit_digits asked for and supported)."""
        rc = -7
        if emit_digits:
            rc = _lib.lib.sbvr_allreduce_add_rmsnorm_digits_f16(
                self.bufs_dev.data_ptr(), self.flags_dev.data_ptr(), self.step.data_ptr(), self.calls_per_step, call_idx,
                self.rank, self.world, self.buf_elems, h.data_ptr(), weight.data_ptr(), h.data_ptr(), y.data_ptr(), rows,
                self.hidden, eps, 1, ws.handle, stream)
            if rc == 0:
                return True
            if rc not in (-7, -5):
                _lib.check(rc, "sbvr_allreduce_add_rmsnorm_digits_f16")
        _lib.check(_lib.lib.sbvr_allreduce_add_rmsnorm_f16(
            self.bufs_dev.data_ptr(), self.flags_dev.data_ptr(), self.step.data_ptr(), self.calls_per_step, call_idx,
            self.rank, self.world, self.buf_elems, h.data_ptr(), weight.data_ptr(), h.data_ptr(), y.data_ptr(), rows,
            self.hidden, eps, ws.handle, stream), "sbvr_allreduce_add_rmsnorm_f16")
        return False

    def push_linear(self, call_idx: int, x_op: int, x: torch.Tensor, w, rows: int, bias=None) -> bool:
        """The row-parallel linear of call `call_idx`, its result pushed to every rank's receive area.  False (nothing
        launched) where the decode GEMV does not apply: the caller then uses partial_out + reduce_add_rmsnorm."""
        from sbvr.core import _cuda_index, _ptr
        if rows > self.push_rows or not x.is_contiguous() or w.out_features != self.hidden:
            return False
        Kp = w.in_features_padded
        if int(w.original_data_shape[-1]) != Kp:
            return False
        b, ix, ib, c, C = w._abi_args()
        di = _cuda_index(w.bvr.device)
        with torch.cuda.device(di):
            st = torch.cuda.current_stream().cuda_stream
            ws = _lib.workspace(di, st)
            rc = _lib.lib.sbvr_linear_push_f16(x_op, x.data_ptr(), None, None, None, 0.0, b, ix, ib, c, C, _ptr(bias),
                                               self.push_descs.data_ptr() + call_idx * self.push_desc_bytes, rows,
                                               self.hidden, Kp, w.num_sums, w.bvr_len, ws.handle, st)
        if rc == -7:
            return False
        _lib.check(rc, "sbvr_linear_push_f16")
        return True

    def ll_reduce_add_rmsnorm(self, call_idx: int, h: torch.Tensor, weight: torch.Tensor, y: torch.Tensor, rows: int,
                              eps: float, ws, stream: int, emit_digits: bool = False) -> bool:
        """Must be the launch directly behind push_linear(call_idx, ...) on the stream: it does not wait for that linear
        to end (h and the norm weight are final long before it).  Returns whether the digits were written."""
        if emit_digits:
            rc = _lib.lib.sbvr_ll_reduce_add_rmsnorm_digits_f16(
                self.recv_local, self.step.data_ptr(), self.calls_per_step, call_idx, self.world, self.push_rows,
                h.data_ptr(), weight.data_ptr(), h.data_ptr(), y.data_ptr(), rows, self.hidden, eps, 1, 1, ws.handle, stream)
            if rc == 0:
                return True
            if rc not in (-7, -5):
                _lib.check(rc, "sbvr_ll_reduce_add_rmsnorm_digits_f16")
        _lib.check(_lib.lib.sbvr_ll_reduce_add_rmsnorm_f16(
            self.recv_local, self.step.data_ptr(), self.calls_per_step, call_idx, self.world, self.push_rows,
            h.data_ptr(), weight.data_ptr(), h.data_ptr(), y.data_ptr(), rows, self.hidden, eps, 1, ws.handle, stream),
            "sbvr_ll_reduce_add_rmsnorm_f16")
        return False

    def end_step(self):
        self.step.add_(1)
