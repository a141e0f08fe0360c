"""ctypes binding of libsbvr_b200.so (the C ABI declared in include/sbvr_b200.h).

There is no fallback: if the library is missing, importing this module raises; if a call
returns a non-zero status, a RuntimeError carrying `sbvr_strerror` is raised, as the reference
binding raised RuntimeError from `std::runtime_error` (reference sbvr/kernels/sbvr_kernel.cu:624-628).
"""
from __future__ import annotations

import ctypes
import os

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_ROOT, "lib", "libsbvr_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: build it with `python sbvr-cpu-arm_b200/build.py` "
        "(there is no CPU or PyTorch fallback for the SBVR kernels)")

lib = ctypes.CDLL(LIB_PATH)

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_ip = ctypes.POINTER(ctypes.c_int)

lib.sbvr_strerror.argtypes = [_i]
lib.sbvr_strerror.restype = ctypes.c_char_p
lib.sbvr_last_cuda_error.argtypes = []
lib.sbvr_last_cuda_error.restype = _i
lib.sbvr_last_timeout_where.argtypes = []
lib.sbvr_last_timeout_where.restype = ctypes.c_uint
lib.sbvr_last_timeout_info.argtypes = [_i]
lib.sbvr_last_timeout_info.restype = ctypes.c_uint
lib.sbvr_query.argtypes = [_i, _ip, _ip, _ip, _ip, _ip]
lib.sbvr_query.restype = _i
lib.sbvr_workspace_create.argtypes = [ctypes.POINTER(_vp), _i, _sz]
lib.sbvr_workspace_create.restype = _i
lib.sbvr_workspace_bytes.argtypes = [_i, _i, _i, _i, ctypes.POINTER(_sz)]
lib.sbvr_workspace_bytes.restype = _i
lib.sbvr_workspace_destroy.argtypes = [_vp]
lib.sbvr_workspace_destroy.restype = _i
lib.sbvr_workspace_status.argtypes = [_vp, _vp]
lib.sbvr_workspace_status.restype = _i
lib.sbvr_decode_f16.argtypes = [_vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp]
lib.sbvr_decode_f16.restype = _i
lib.sbvr_linear_f16.argtypes = [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]
lib.sbvr_linear_f16.restype = _i
lib.sbvr_linear_fused_f16.argtypes = [_i, _vp, _vp, _vp, _vp, ctypes.c_float, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i,
                                      _i, _i, _vp, _vp]
lib.sbvr_linear_fused_f16.restype = _i
lib.sbvr_popc_mm_f16.argtypes = [_vp, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]
lib.sbvr_popc_mm_f16.restype = _i
lib.sbvr_linear_t_f16.argtypes = [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]
lib.sbvr_linear_t_f16.restype = _i
lib.sbvr_encode_mse_f16.argtypes = [_vp, _i, _vp, _i, _i, _vp, _vp]
lib.sbvr_encode_mse_f16.restype = _i
lib.sbvr_encode_select_f16.argtypes = [_vp, _i, _vp, _vp, _i, _vp, _vp]
lib.sbvr_encode_select_f16.restype = _i
lib.sbvr_encode_pack.argtypes = [_vp, _i, _i, _i, _vp, _vp]
lib.sbvr_encode_pack.restype = _i
lib.sbvr_linear_f16_host.argtypes = [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]
lib.sbvr_linear_f16_host.restype = _i
lib.sbvr_linear_f16_noalloc.argtypes = [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp]
lib.sbvr_linear_f16_noalloc.restype = _i

_f = ctypes.c_float
lib.sbvr_add_rmsnorm_f16.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]
lib.sbvr_add_rmsnorm_f16.restype = _i
lib.sbvr_rope_append_f16.argtypes = [_vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]
lib.sbvr_rope_append_f16.restype = _i
lib.sbvr_attention_f16.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp]
lib.sbvr_attention_f16.restype = _i
lib.sbvr_rope_attention_f16.argtypes = [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp]
lib.sbvr_rope_attention_f16.restype = _i
lib.sbvr_silu_mul_f16.argtypes = [_vp, _vp, _i, _i, _vp]
lib.sbvr_silu_mul_f16.restype = _i
lib.sbvr_embedding_f16.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
lib.sbvr_embedding_f16.restype = _i
lib.sbvr_argmax_f16.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
lib.sbvr_argmax_f16.restype = _i

lib.sbvr_allreduce_add_rmsnorm_f16.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _sz, _vp, _vp, _vp, _vp, _i, _i, _f, _vp, _vp]
lib.sbvr_allreduce_add_rmsnorm_f16.restype = _i
lib.sbvr_linear_push_f16.argtypes = [_i, _vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]
lib.sbvr_linear_push_f16.restype = _i
lib.sbvr_ll_reduce_add_rmsnorm_f16.argtypes = [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _vp]
lib.sbvr_ll_reduce_add_rmsnorm_f16.restype = _i
lib.sbvr_ll_reduce_add_rmsnorm_digits_f16.argtypes = [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _vp, _vp]
lib.sbvr_ll_reduce_add_rmsnorm_digits_f16.restype = _i
lib.sbvr_allreduce_add_rmsnorm_digits_f16.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _sz, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _vp]
lib.sbvr_allreduce_add_rmsnorm_digits_f16.restype = _i

EXPORTS = ["sbvr_popc_mm_f16", "sbvr_linear_t_f16", "sbvr_encode_mse_f16", "sbvr_encode_select_f16", "sbvr_encode_pack", "sbvr_rope_attention_f16", "sbvr_linear_fused_f16", "sbvr_allreduce_add_rmsnorm_f16", "sbvr_linear_push_f16", "sbvr_ll_reduce_add_rmsnorm_f16", "sbvr_ll_reduce_add_rmsnorm_digits_f16", "sbvr_allreduce_add_rmsnorm_digits_f16", "sbvr_add_rmsnorm_f16", "sbvr_rope_append_f16", "sbvr_attention_f16", "sbvr_silu_mul_f16",
           "sbvr_embedding_f16", "sbvr_argmax_f16", "sbvr_linear_f16_noalloc", "sbvr_workspace_bytes", "sbvr_strerror", "sbvr_last_cuda_error", "sbvr_last_timeout_where", "sbvr_last_timeout_info", "sbvr_query", "sbvr_workspace_create",
           "sbvr_workspace_destroy", "sbvr_workspace_status", "sbvr_decode_f16", "sbvr_linear_f16",
           "sbvr_linear_f16_host"]


class PushDesc(ctypes.Structure):
    """sbvr_push_desc_t of include/sbvr_b200.h."""
    _fields_ = [("peer_recv", ctypes.c_ulonglong * 16), ("step", ctypes.c_void_p), ("calls_per_step", ctypes.c_int),
                ("call_idx", ctypes.c_int), ("rank", ctypes.c_int), ("world", ctypes.c_int), ("rows_max", ctypes.c_int),
                ("reserved", ctypes.c_int)]


def strerror(rc: int) -> str:
    return lib.sbvr_strerror(rc).decode()


def check(rc: int, what: str = "sbvr") -> None:
    if rc != 0:
        extra = ""
        if rc == -4:
            extra = f" (cudaError {lib.sbvr_last_cuda_error()})"
        raise RuntimeError(f"{what}: {strerror(rc)}{extra}")


def query(device: int = 0) -> dict:
    vals = [ctypes.c_int(0) for _ in range(5)]
    check(lib.sbvr_query(device, *[ctypes.byref(v) for v in vals]), "sbvr_query")
    keys = ["sm_count", "smem_per_block_optin", "l2_bytes", "cc_major", "cc_minor"]
    return {k: v.value for k, v in zip(keys, vals)}


class Workspace:
    """Owns one `sbvr_workspace_t`: the device status word of the kernels' bounded waits, the re-tiled
    activations and split-K partial sums of the batched kernel, staging buffers of the host-pointer call."""

    DEFAULT_BYTES = 32 << 20

    def __init__(self, device: int, nbytes: int = 0):
        self.handle = _vp()
        self.device = device
        self.nbytes = nbytes or self.DEFAULT_BYTES
        check(lib.sbvr_workspace_create(ctypes.byref(self.handle), device, nbytes), "sbvr_workspace_create")

    def status(self, stream: int) -> int:
        return lib.sbvr_workspace_status(self.handle, _vp(stream))

    def close(self):
        if self.handle:
            lib.sbvr_workspace_destroy(self.handle)
            self.handle = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_workspaces: dict = {}
# Workspaces replaced by larger ones.  They are never freed: a captured CUDA graph keeps the raw pointers of the
# workspace its kernels were recorded with (status word, counters, scratch), and would write into freed memory
# on replay if the replaced allocation went back to the driver.
_retired: list = []


def workspace_bytes(device: int, M: int, N: int, K: int) -> int:
    out = _sz(0)
    check(lib.sbvr_workspace_bytes(device, M, N, K, ctypes.byref(out)), "sbvr_workspace_bytes")
    return out.value


def workspace(device: int, stream: int, nbytes: int = 0) -> Workspace:
    """One workspace per (device, stream): calls on one stream are ordered, so they may share scratch.
    A workspace smaller than `nbytes` is replaced by a larger one; the old one stays allocated for the life of the
    process (graphs captured earlier on this stream still point into it)."""
    key = (device, stream)
    ws = _workspaces.get(key)
    if ws is not None and ws.nbytes < nbytes:
        _retired.append(ws)
        ws = None
    if ws is None:
        ws = Workspace(device, max(nbytes, Workspace.DEFAULT_BYTES))
        _workspaces[key] = ws
    return ws
