"""TEST INFRASTRUCTURE - ctypes loader of oracle/_ref/libsbvr_ref_cuda.so, the REFERENCE's own CUDA kernels
(sbvr/kernels/sbvr_kernel.cu, compiled unchanged by `make -C oracle ref REF=<checkout>`) behind the C shim
oracle/ref_cuda_shim.cu.  Only tests and the benchmark's comparator leg import this; the product never does.

`lib()` returns None when the library has not been built (no reference checkout at build time).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(_HERE, "_ref", "libsbvr_ref_cuda.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(PATH):
            return None
        L = ctypes.CDLL(PATH)
        vp, i = ctypes.c_void_p, ctypes.c_int
        L.sbvr_ref_init.argtypes, L.sbvr_ref_init.restype = [], i
        L.sbvr_ref_row_deq_mm_T.argtypes = [vp] * 6 + [i] * 7
        L.sbvr_ref_row_deq_mm_T.restype = i
        L.sbvr_ref_mm_T.argtypes = [vp] * 8 + [i] * 8
        L.sbvr_ref_mm_T.restype = i
        L.sbvr_ref_time_us.argtypes = [i, i] + [vp] * 8 + [i] * 8
        L.sbvr_ref_time_us.restype = ctypes.c_float
        if L.sbvr_ref_init() < 1:
            return None
        _lib = L
    return _lib


def _p(t):
    return None if t is None else t.data_ptr()


def row_deq_mm_T(x, bvr_t, idx, cache, bias=None, use_shfl=0):
    """The reference's `_sbvr_row_deq_mm_T` (sbvr/kernels/sbvr_ops.cpp:79-120) on CUDA tensors: x fp16 [M, K], bvr_t uint32/int32
    [N/32, K, S], idx uint8|uint16 [N/256, K], cache fp16 [C, S].  Its S = 4 kernel computes the first row of x only."""
    import torch
    M, K = x.shape
    N, S, C = bvr_t.shape[0] * 32, bvr_t.shape[2], cache.shape[0]
    out = torch.zeros((M, N), dtype=torch.float16, device=x.device)
    torch.cuda.synchronize()
    rc = lib().sbvr_ref_row_deq_mm_T(_p(x), _p(bvr_t), _p(idx), _p(cache), _p(bias), _p(out), M, N, K, S, C, use_shfl,
                                     x.device.index or 0)
    if rc != 0:
        raise RuntimeError(f"reference row_deq kernel: cudaError {rc}")
    return out


def mm_T(l_bvr, l_idx, l_cache, r_bvr, r_idx, r_cache, bias=None):
    """The reference's `_sbvr_mm_T` (sbvr/kernels/sbvr_ops.cpp:35-76): both operands encoded, bvr [K/32, rows, S]."""
    import torch
    Kw, M, LS = l_bvr.shape
    N, RS = r_bvr.shape[1], r_bvr.shape[2]
    out = torch.zeros((M, N), dtype=torch.float16, device=l_bvr.device)
    torch.cuda.synchronize()
    rc = lib().sbvr_ref_mm_T(_p(l_bvr), _p(l_idx), _p(l_cache), _p(r_bvr), _p(r_idx), _p(r_cache), _p(bias), _p(out), M, N, Kw,
                             LS, RS, l_cache.shape[0], r_cache.shape[0], l_bvr.device.index or 0)
    if rc != 0:
        raise RuntimeError(f"reference mm_T kernel: cudaError {rc}")
    return out


def time_row_deq_us(x, bvr_t, idx, cache, reps=20):
    import torch
    M, K = x.shape
    N, S, C = bvr_t.shape[0] * 32, bvr_t.shape[2], cache.shape[0]
    out = torch.zeros((M, N), dtype=torch.float16, device=x.device)
    torch.cuda.synchronize()
    return float(lib().sbvr_ref_time_us(0, reps, _p(x), _p(bvr_t), _p(idx), _p(cache), None, None, None, _p(out), M, N, K, S, 0,
                                        C, 0, x.device.index or 0))


def time_mm_T_us(l_bvr, l_idx, l_cache, r_bvr, r_idx, r_cache, reps=20):
    import torch
    Kw, M, LS = l_bvr.shape
    N, RS = r_bvr.shape[1], r_bvr.shape[2]
    out = torch.zeros((M, N), dtype=torch.float16, device=l_bvr.device)
    torch.cuda.synchronize()
    return float(lib().sbvr_ref_time_us(1, reps, _p(l_bvr), _p(l_idx), _p(l_cache), _p(r_bvr), _p(r_idx), _p(r_cache), None,
                                        _p(out), M, N, Kw, LS, RS, l_cache.shape[0], r_cache.shape[0],
                                        l_bvr.device.index or 0))
