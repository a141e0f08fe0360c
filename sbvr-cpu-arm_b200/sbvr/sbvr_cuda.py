"""Raw-tensor entry points with the names and argument order of the reference's CUDA extension module
(`sbvr_cuda`, sbvr/kernels/sbvr_ops.cpp:151-171), so that call sites written against it
(`sbvr.sbvr_cuda._sbvr_row_deq_mm_T(x, bvr, idx, cache, bias, use_shfl)`, test_sbvr.py:322-325, :588-592) run unchanged.
Shapes are inferred from the tensors exactly as the binding does (sbvr_ops.cpp:45-51, :93-97); "no bias" is a tensor
whose length is not N (:56-58, :102-104)."""
from __future__ import annotations

import torch

from . import _lib


def _dev_index(t: torch.Tensor) -> int:
    if t.device.type != "cuda":
        raise ValueError("tensors must live on a CUDA device")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _idx_bytes(idx: torch.Tensor, cache: torch.Tensor) -> int:
    # the reference picks the index width from the codebook size (sbvr/kernels/sbvr_kernel.cu:887, :931-932)
    ib = 1 if cache.shape[0] <= 256 else 2
    if idx.element_size() != ib:
        raise ValueError(f"coefficient index must be {'uint8' if ib == 1 else 'uint16'} for {cache.shape[0]} cache lines")
    return ib


def _sbvr_cuda_init() -> None:
    """The reference caches device 0's properties here (sbvr_ops.cpp:153); this library reads them on first use."""
    _lib.query(torch.cuda.current_device())


@torch.inference_mode()
def _sbvr_row_deq_mm_T(l_w: torch.Tensor, r_bvr: torch.Tensor, r_coeff_idx: torch.Tensor, r_coeff_cache: torch.Tensor,
                       bias: torch.Tensor, use_shfl: int = 0) -> torch.Tensor:
    """out[M, N] = l_w[M, K] @ W^T + bias with the weight in the transposed encoding: r_bvr uint32 [N/32, K, S],
    r_coeff_idx [N/256, K], r_coeff_cache fp16 [C, S] (reference sbvr_row_deq_mm_T, sbvr_ops.cpp:79-120).
    `use_shfl` selected between two reference kernels with the same result; it is accepted and ignored."""
    if l_w.dtype != torch.float16 or r_coeff_cache.dtype != torch.float16:
        raise ValueError("activations and coefficients must be float16")
    if r_bvr.dtype == torch.int32:
        r_bvr = r_bvr.view(torch.uint32)
    if r_bvr.dtype != torch.uint32 or r_bvr.dim() != 3:
        raise ValueError("r_bvr must be uint32 [N/32, K, S]")
    di = _dev_index(l_w)
    M, K = int(l_w.shape[0]), int(r_bvr.shape[1])
    N, S, C = int(r_bvr.shape[0]) * 32, int(r_bvr.shape[2]), int(r_coeff_cache.shape[0])
    if l_w.shape[1] != K:
        raise ValueError(f"inner dimension mismatch: activation {l_w.shape[1]}, weight {K}")
    G = N // int(r_coeff_idx.shape[0])
    ib = _idx_bytes(r_coeff_idx, r_coeff_cache)
    l_w, r_bvr, r_coeff_idx, r_coeff_cache = (t.contiguous() for t in (l_w, r_bvr, r_coeff_idx, r_coeff_cache))
    b = bias.contiguous() if (bias is not None and bias.numel() == N) else None
    out = torch.empty((M, N), dtype=torch.float16, device=l_w.device)
    if M == 0:
        return out
    with torch.cuda.device(di):
        st = torch.cuda.current_stream().cuda_stream
        ws = _lib.workspace(di, st)
        _lib.check(_lib.lib.sbvr_linear_t_f16(l_w.data_ptr(), r_bvr.data_ptr(), r_coeff_idx.data_ptr(), ib,
                                              r_coeff_cache.data_ptr(), C, None if b is None else b.data_ptr(),
                                              out.data_ptr(), M, N, K, S, G, ws.handle, st), "sbvr_linear_t_f16")
    return out


@torch.inference_mode()
def _sbvr_mm_T(l_bvr: torch.Tensor, l_coeff_idx: torch.Tensor, l_coeff_cache: torch.Tensor, r_bvr: torch.Tensor,
               r_coeff_idx: torch.Tensor, r_coeff_cache: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[M, N] with both operands SBVR-encoded, l_bvr uint32 [K/32, M, LS], r_bvr uint32 [K/32, N, RS]
    (reference sbvr_mm_T, sbvr_ops.cpp:35-76)."""
    if l_bvr.dtype == torch.int32:
        l_bvr = l_bvr.view(torch.uint32)
    if r_bvr.dtype == torch.int32:
        r_bvr = r_bvr.view(torch.uint32)
    di = _dev_index(l_bvr)
    M, N, K = int(l_bvr.shape[1]), int(r_bvr.shape[1]), int(r_bvr.shape[0]) * 32
    if int(l_bvr.shape[0]) * 32 != K:
        raise ValueError("inner dimension mismatch")
    lib_, rib = _idx_bytes(l_coeff_idx, l_coeff_cache), _idx_bytes(r_coeff_idx, r_coeff_cache)
    ts = [t.contiguous() for t in (l_bvr, l_coeff_idx, l_coeff_cache, r_bvr, r_coeff_idx, r_coeff_cache)]
    b = bias.contiguous() if (bias is not None and bias.numel() == N) else None
    out = torch.empty((M, N), dtype=torch.float16, device=l_bvr.device)
    with torch.cuda.device(di):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib.sbvr_popc_mm_f16(ts[0].data_ptr(), ts[1].data_ptr(), lib_, ts[2].data_ptr(),
                                             int(ts[2].shape[0]), int(ts[0].shape[2]), ts[3].data_ptr(), ts[4].data_ptr(),
                                             rib, ts[5].data_ptr(), int(ts[5].shape[0]), int(ts[3].shape[2]),
                                             None if b is None else b.data_ptr(), out.data_ptr(), M, N, K, st),
                   "sbvr_popc_mm_f16")
    return out
