"""Host side of the SBVR tensor format on B200: the `sbvr` container, its serialized form,
`load`, `linear` and `mm_T`.

Mirrors the public surface of the reference's `sbvr/core.py` (class `sbvr` :205-317,
`_sbvr_serialized` :62-201, `decode` :926-949, `save` :918-924, `load` :1041-1050, `mm_T`
:1029-1039) on the same packed tensors, so files written by the reference load here and call
sites keep working.  All arithmetic runs in the CUDA library behind `_lib`; nothing in this
module computes on the CPU and there is no fallback when the library or a GPU is missing.

Packed tensors (GPU layout of the reference, sbvr/core.py:724-805):
    bvr         uint32 [Kp/32, N, S]
    coeff_idx   uint8 | uint16 [Kp/G, N]
    coeff_cache float16 [C, S]
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import _lib

BVR_LEN = 256          # group length the reference enforces (sbvr/core.py:222)


def _r_str(s):
    return "\033[91m" + str(s) + "\033[0m"


class _sbvr_serialized:
    """Pickle-compatible with the reference class of the same qualified name
    (sbvr/core.py:62-201): tensors are kept as int8 byte views next to their shape and dtype."""

    def __init__(self, num_sums: int, bvr_len: int, compute_dtype: torch.dtype, bvr_dtype: torch.dtype,
                 original_dtype: torch.dtype, original_data_shape, bvr: torch.Tensor, coeff_idx: torch.Tensor,
                 coeff_cache: torch.Tensor, input_num_sums: int = -1, input_coeff: Optional[torch.Tensor] = None):
        self.num_sums = num_sums
        self.bvr_len = bvr_len
        self.compute_dtype = compute_dtype
        self.bvr_dtype = bvr_dtype
        word_bits = torch.tensor(0, dtype=bvr_dtype).element_size() * 8
        if num_sums > 11 and compute_dtype == torch.float16:
            raise UserWarning(_r_str("Warning: compute_dtype float16 does not have sufficient precision "
                                     "for num_sums > 11."))
        if bvr_len % word_bits != 0:
            raise ValueError(_r_str("BVR length must be a multiple of ") + f"{word_bits}")
        self.original_dtype = original_dtype
        self.original_data_shape = original_data_shape
        padded = list(original_data_shape)
        padded[-1] = (padded[-1] + bvr_len - 1) // bvr_len * bvr_len
        self.padded_data_shape = padded
        if bvr.dtype != bvr_dtype:
            raise ValueError(_r_str(f"The BVR data type does not match - expected type {bvr_dtype} "
                                    f"but got {bvr.dtype}"))
        lines = coeff_cache.shape[0]
        if lines <= 256:
            if coeff_idx.dtype != torch.uint8:
                raise ValueError(_r_str(f"The coefficient index data type must be uint8 but got "
                                        f"{coeff_idx.dtype}, number of cache lines: {lines}"))
        elif lines <= 65536:
            if coeff_idx.dtype != torch.uint16:
                raise ValueError(_r_str(f"The coefficient index data type must be uint16 but got "
                                        f"{coeff_idx.dtype}, number of cache lines: {lines}"))
        else:
            raise ValueError(_r_str(f"Unsupported number of cache lines, {lines}"))
        if coeff_cache.dtype != compute_dtype:
            raise ValueError(_r_str(f"The coefficient cache data type does not match - expected type "
                                    f"{compute_dtype} but got {coeff_cache.dtype}"))
        self.bvr = self._serialize_tensor(bvr)
        self.bvr_shape = bvr.shape
        self.bvr_dtype = bvr.dtype
        self.coeff_idx = self._serialize_tensor(coeff_idx)
        self.coeff_idx_shape = coeff_idx.shape
        self.coeff_idx_dtype = coeff_idx.dtype
        self.coeff_cache = self._serialize_tensor(coeff_cache)
        self.coeff_cache_shape = coeff_cache.shape
        self.coeff_cache_dtype = coeff_cache.dtype
        self.input_num_sums = input_num_sums
        if input_coeff is not None:
            if input_coeff.dtype != compute_dtype:
                raise ValueError(_r_str("The input coefficient data type does not match"))
            self.input_coeff = self._serialize_tensor(input_coeff)
            self.input_coeff_shape = input_coeff.shape
            self.input_coeff_dtype = input_coeff.dtype
        else:
            self.input_coeff = None
            self.input_coeff_shape = None
            self.input_coeff_dtype = None

    @staticmethod
    def _serialize_tensor(t: torch.Tensor) -> torch.Tensor:
        flat = t.detach().cpu().contiguous().reshape(-1)
        return flat.view(torch.int8).clone()

    @staticmethod
    def _deserialize_tensor(raw: torch.Tensor, shape, dtype) -> torch.Tensor:
        if str(dtype) not in ("torch.uint8", "torch.uint16", "torch.uint32", "torch.int32", "torch.float16",
                              "torch.float32"):
            raise ValueError(f"Unsupported dtype: {dtype}")
        return raw.detach().cpu().contiguous().view(dtype).reshape(tuple(shape)).clone()

    def deserialize_sbvr(self):
        bvr = self._deserialize_tensor(self.bvr, self.bvr_shape, self.bvr_dtype)
        idx = self._deserialize_tensor(self.coeff_idx, self.coeff_idx_shape, self.coeff_idx_dtype)
        cache = self._deserialize_tensor(self.coeff_cache, self.coeff_cache_shape, self.coeff_cache_dtype)
        inp = None
        if self.input_coeff is not None:
            inp = self._deserialize_tensor(self.input_coeff, self.input_coeff_shape, self.input_coeff_dtype)
        return (self.num_sums, self.bvr_len, self.compute_dtype, self.bvr_dtype, self.original_dtype,
                self.original_data_shape, bvr, idx, cache, self.input_num_sums, inp)


def _cuda_index(dev: torch.device) -> int:
    if dev.type != "cuda":
        raise RuntimeError("SBVR kernels run on CUDA tensors only (there is no CPU path); got device " + str(dev))
    return dev.index if dev.index is not None else torch.cuda.current_device()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class sbvr(torch.nn.Module):
    """A weight held as packed bit-planes + coefficient codebook (reference class `sbvr`,
    sbvr/core.py:205-317).  Construct it from a serialized object (what `load` does) or from packed
    tensors with `sbvr.from_packed`.  `group_len` (the reference's `bvr_len`) is 256 for anything the
    reference wrote; `from_packed` also accepts 128 and a direct per-group coefficient tensor."""

    def __init__(self, data: torch.Tensor = None, encoder_config: dict = None, device: torch.device = None,
                 sbvr_serialized: _sbvr_serialized = None, verbose_level: int = 1, trans: bool = False,
                 cpu_kernel: bool = False, cpu_kernel_v2: bool = False, gpu_tensor_gen: bool = False):
        super().__init__()
        self.verbose_level = verbose_level
        if data is not None and sbvr_serialized is not None:
            raise ValueError(_r_str("Cannot provide both data and serialized SBVR"))
        if data is None and sbvr_serialized is None:
            raise ValueError(_r_str("Must provide either data or serialized SBVR"))
        if cpu_kernel or cpu_kernel_v2:
            raise ValueError(_r_str("The ARM CPU tensor layouts (cpu_kernel / cpu_kernel_v2) are not supported: "
                                    "this build runs the GPU layout on B200 only"))
        if data is not None:
            self._encode(data, encoder_config, device, trans)
            return
        if not isinstance(sbvr_serialized, _sbvr_serialized):
            raise ValueError(_r_str("Serialized SBVR object is not valid"))
        _device = device if device is not None else torch.device("cuda")
        (self.num_sums, self.bvr_len, self.compute_dtype, self.bvr_dtype, self.original_dtype,
         self.original_data_shape, bvr, coeff_idx, coeff_cache, self.input_num_sums,
         input_coeff) = sbvr_serialized.deserialize_sbvr()
        if self.bvr_len != BVR_LEN:
            raise ValueError(_r_str(f"bvr length does not match the enforced value, expected {BVR_LEN} "
                                    f"but got {self.bvr_len}"))
        if self.compute_dtype != torch.float16:
            raise ValueError(_r_str(f"Compute data type does not match the enforced value, expected "
                                    f"{torch.float16} but got {self.compute_dtype}"))
        if self.bvr_dtype != torch.uint32:
            raise ValueError(_r_str(f"BVR data type does not match the enforced value, expected "
                                    f"{torch.uint32} but got {self.bvr_dtype}"))
        self._install(bvr, coeff_idx, coeff_cache, _device)
        self.input_coeff = None if input_coeff is None else torch.nn.Parameter(input_coeff.to(_device),
                                                                               requires_grad=False)

    # -- construction ---------------------------------------------------------------------
    def _encode(self, data, encoder_config, device, trans):
        """`sbvr(data, encoder_config)` (reference sbvr/core.py:243-276): encode a dense tensor on the GPU.  `trans=True`
        encodes the transpose (groups along the other dimension), as there (:244-245)."""
        from . import encoder
        if not isinstance(data, torch.Tensor):
            raise ValueError(_r_str("Data must be a torch tensor"))
        if trans:
            data = data.transpose(0, 1).contiguous()
        conf = encoder.EncoderConfig.from_dict(encoder_config)
        dev = torch.device(device) if device is not None else torch.device("cuda")
        self.num_sums, self.bvr_len = conf.num_sums, BVR_LEN
        self.compute_dtype, self.bvr_dtype = torch.float16, torch.uint32
        self.original_dtype, self.original_data_shape = data.dtype, data.shape
        self.input_num_sums, self.input_coeff = -1, None
        bvr, idx, cache, self.encoder_stats = encoder.encode(data, conf, dev)
        self._install(bvr, idx, cache, dev)
        if self.verbose_level > 0:
            print(f"Encoding complete. {self.encoder_stats}")
            print(self.get_sbvr_info())

    def _install(self, bvr, coeff_idx, coeff_cache, device):
        self.bvr = torch.nn.Parameter(bvr.to(device).contiguous(), requires_grad=False)
        self.coeff_idx = None if coeff_idx is None else torch.nn.Parameter(coeff_idx.to(device).contiguous(),
                                                                           requires_grad=False)
        self.coeff_cache = torch.nn.Parameter(coeff_cache.to(device).contiguous(), requires_grad=False)

    @classmethod
    def from_packed(cls, bvr: torch.Tensor, coeff_idx: Optional[torch.Tensor], coeff: torch.Tensor,
                    original_shape=None, group_len: int = BVR_LEN, device=None, verbose_level: int = 0) -> "sbvr":
        """Wrap already packed tensors.  `coeff_idx=None` means `coeff` is the direct form
        [Kp/group_len, N, S]; otherwise `coeff` is the codebook [C, S]."""
        self = cls.__new__(cls)
        torch.nn.Module.__init__(self)
        self.verbose_level = verbose_level
        KW, N, S = bvr.shape
        self.num_sums, self.bvr_len = int(S), int(group_len)
        self.compute_dtype, self.bvr_dtype, self.original_dtype = torch.float16, torch.uint32, torch.float16
        self.original_data_shape = torch.Size(original_shape) if original_shape is not None else torch.Size((N, KW * 32))
        self.input_num_sums, self.input_coeff = -1, None
        if bvr.dtype == torch.int32:
            bvr = bvr.view(torch.uint32)
        if bvr.dtype != torch.uint32 or coeff.dtype != torch.float16:
            raise ValueError(_r_str("bvr must be uint32 and coefficients float16"))
        if (KW * 32) % group_len:
            raise ValueError(_r_str("padded inner length must be a multiple of the group length"))
        if coeff_idx is not None:
            want = torch.uint8 if coeff.shape[0] <= 256 else torch.uint16
            if coeff_idx.dtype == torch.int16:
                coeff_idx = coeff_idx.view(torch.uint16)
            if coeff_idx.dtype != want:
                raise ValueError(_r_str(f"The coefficient index data type must be {want} but got {coeff_idx.dtype}, "
                                        f"number of cache lines: {coeff.shape[0]}"))
        dev = device if device is not None else bvr.device
        self._install(bvr, coeff_idx, coeff, dev)
        return self

    # -- shape helpers (reference sbvr/core.py:319-343) --------------------------------------
    def _get_bvr_num_bits(self):
        return 32

    def _get_padded_data_shape(self):
        s = list(self.original_data_shape)
        s[-1] = (s[-1] + self.bvr_len - 1) // self.bvr_len * self.bvr_len
        return torch.Size(s)

    def _get_dummy_bias(self):
        return torch.zeros([0], dtype=self.compute_dtype, device=self.coeff_cache.device)

    @property
    def out_features(self) -> int:
        return int(self.bvr.shape[1])

    @property
    def in_features_padded(self) -> int:
        return int(self.bvr.shape[0]) * 32

    def _abi_args(self):
        """(bvr_ptr, idx_ptr, idx_bytes, coeff_ptr, C) for the C ABI."""
        if self.coeff_idx is None:
            return self.bvr.data_ptr(), None, 0, self.coeff_cache.data_ptr(), 0
        ib = self.coeff_idx.element_size()
        # the reference picks the index width from the codebook size (sbvr/kernels/sbvr_kernel.cu:887)
        assert ib == (1 if self.coeff_cache.shape[0] <= 256 else 2), "coeff_idx dtype disagrees with codebook size"
        return self.bvr.data_ptr(), self.coeff_idx.data_ptr(), ib, self.coeff_cache.data_ptr(), int(
            self.coeff_cache.shape[0])

    # -- operations ---------------------------------------------------------------------------
    @torch.inference_mode()
    def decode(self) -> torch.Tensor:
        """Dense fp16 tensor of the original shape (reference `decode`, sbvr/core.py:926-949), computed by
        the CUDA decode kernel, bit-exact with the reference."""
        dev = self.bvr.device
        di = _cuda_index(dev)
        N, Kp = self.out_features, self.in_features_padded
        K = int(self.original_data_shape[-1])
        out = torch.empty((N, K), dtype=torch.float16, device=dev)
        b, ix, ib, c, C = self._abi_args()
        with torch.cuda.device(di):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.lib.sbvr_decode_f16(b, ix, ib, c, C, out.data_ptr(), K, N, Kp, K, self.num_sums,
                                                self.bvr_len, st), "sbvr_decode_f16")
        return out.view(self.original_data_shape) if out.numel() == int(np.prod(self.original_data_shape)) else out

    def _serialize(self) -> _sbvr_serialized:
        if self.coeff_idx is None:
            raise ValueError(_r_str("the direct-coefficient form has no serialized representation"))
        return _sbvr_serialized(self.num_sums, self.bvr_len, self.compute_dtype, self.bvr_dtype, self.original_dtype,
                                self.original_data_shape, self.bvr, self.coeff_idx, self.coeff_cache,
                                self.input_num_sums, self.input_coeff)

    @torch.inference_mode()
    def save(self, filename):
        torch.save(self._serialize(), filename)

    def get_sbvr_info(self) -> str:
        return (f"SBVR Info: num_sums={self.num_sums} bvr_len={self.bvr_len} "
                f"original_shape={tuple(self.original_data_shape)} bvr={tuple(self.bvr.shape)} "
                f"coeff_idx={None if self.coeff_idx is None else tuple(self.coeff_idx.shape)} "
                f"coeff_cache={tuple(self.coeff_cache.shape)}")


@torch.inference_mode()
def linear(x: torch.Tensor, w: sbvr, bias: Optional[torch.Tensor] = None, algo: int = 0,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ W.T (+ bias) with fp16 `x` [..., K] and a packed weight `w`, fp32 accumulation, fp16 result.

    The product the reference's Llama flow computes with the decoded weight (sbvr_utils/utils_llama.py:147)
    and its `_sbvr_row_deq_mm_T` binding computes on a transposed encoding (sbvr/kernels/sbvr_ops.cpp:79-120).
    `bias` may be None or an empty tensor (the reference's "no bias" convention, sbvr/core.py:353-358).
    """
    if x.dtype != torch.float16:
        raise ValueError("activations must be float16")
    dev = w.bvr.device
    di = _cuda_index(dev)
    if x.device != dev:
        raise ValueError(f"activation on {x.device}, weight on {dev}")
    K = int(w.original_data_shape[-1])
    Kp, N = w.in_features_padded, w.out_features
    if x.shape[-1] != K:
        raise ValueError(_r_str(f"inner dimension mismatch: activation {x.shape[-1]}, weight {K}"))
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K)
    if Kp != K:
        x2 = torch.nn.functional.pad(x2, (0, Kp - K))
    x2 = x2.contiguous()
    M = x2.shape[0]
    if bias is not None and bias.numel() == 0:
        bias = None
    if bias is not None:
        if bias.numel() != N or bias.dtype != torch.float16:
            raise ValueError("bias must be float16 of length N")
        bias = bias.contiguous()
    y = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=dev)
    if M == 0:
        return y.view(*lead, N)
    b, ix, ib, c, C = w._abi_args()
    with torch.cuda.device(di):
        st = torch.cuda.current_stream().cuda_stream
        ws = _lib.workspace(di, st, _lib.workspace_bytes(di, M, N, Kp) if M > 4 else 0)
        _lib.check(_lib.lib.sbvr_linear_f16(x2.data_ptr(), b, ix, ib, c, C, _ptr(bias), y.data_ptr(), M, N, Kp,
                                            w.num_sums, w.bvr_len, algo, ws.handle, st), "sbvr_linear_f16")
    return y.view(*lead, N)


XOP_NONE, XOP_SILU_MUL, XOP_ADD_RMSNORM, XOP_DIGITS = 0, 1, 2, 3


@torch.inference_mode()
def linear_fused(op: int, x: torch.Tensor, w: sbvr, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
                 norm_weight: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None, eps: float = 0.0,
                 bias: Optional[torch.Tensor] = None) -> bool:
    """Decode linear with the op in front of it folded into the kernel (`sbvr_linear_fused_f16`):
    XOP_SILU_MUL: out = (silu(x[:, :K]) * x[:, K:]) @ W.T;  XOP_ADD_RMSNORM: out = rmsnorm(x + delta) * norm_weight @ W.T
    with x + delta stored to h_out;  XOP_DIGITS: out = x @ W.T where the kernel launched directly before on this stream
    (an all-reduce + RMSNorm with emit_digits) has already left x quantised in the stream's workspace.
    Returns False (and computes nothing) where the decode kernel does not apply."""
    dev = w.bvr.device
    di = _cuda_index(dev)
    Kp, N = w.in_features_padded, w.out_features
    M = x.shape[0]
    if M > 4 or int(w.original_data_shape[-1]) != Kp or not x.is_contiguous():
        return False
    b, ix, ib, c, C = w._abi_args()
    with torch.cuda.device(di):
        st = torch.cuda.current_stream().cuda_stream
        ws = _lib.workspace(di, st)
        rc = _lib.lib.sbvr_linear_fused_f16(op, x.data_ptr(), _ptr(delta), _ptr(norm_weight), _ptr(h_out), float(eps), b,
                                            ix, ib, c, C, _ptr(bias), out.data_ptr(), M, N, Kp, w.num_sums, w.bvr_len,
                                            ws.handle, st)
    if rc == -7:
        return False
    _lib.check(rc, "sbvr_linear_fused_f16")
    return True


@torch.inference_mode()
def mm_T(lhs, rhs: sbvr, bias=None):
    """`lhs @ rhs.T + bias` (reference `mm_T`, sbvr/core.py:1029-1039).  `lhs` may be an fp16 tensor (-> `linear`) or, as
    in the reference, an `sbvr` object: then both operands stay encoded and the product runs on the popcount kernel
    (`sbvr_popc_mm_f16`, the reference's `_sbvr_mm_T`); encodings it does not cover (more than 4 planes, direct
    coefficients, group length other than 256) are decoded on the GPU and go through `linear`."""
    if not isinstance(lhs, sbvr):
        return linear(lhs, rhs, bias)
    ok = (lhs.bvr_len == 256 and rhs.bvr_len == 256 and lhs.coeff_idx is not None and rhs.coeff_idx is not None and
          2 <= lhs.num_sums <= 4 and 2 <= rhs.num_sums <= 4 and lhs.in_features_padded == rhs.in_features_padded and
          lhs.bvr.device == rhs.bvr.device)
    if not ok:
        return linear(lhs.decode(), rhs, bias)
    dev = rhs.bvr.device
    di = _cuda_index(dev)
    M, N, K = lhs.out_features, rhs.out_features, rhs.in_features_padded
    if bias is not None and bias.numel() == 0:
        bias = None
    if bias is not None:
        if bias.numel() != N or bias.dtype != torch.float16:
            raise ValueError("bias must be float16 of length N")
        bias = bias.contiguous()
    y = torch.empty((M, N), dtype=torch.float16, device=dev)
    lb, lix, lib_, lc, lC = lhs._abi_args()
    rb, rix, rib, rc, rC = rhs._abi_args()
    with torch.cuda.device(di):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib.sbvr_popc_mm_f16(lb, lix, lib_, lc, lC, lhs.num_sums, rb, rix, rib, rc, rC, rhs.num_sums,
                                             _ptr(bias), y.data_ptr(), M, N, K, st), "sbvr_popc_mm_f16")
    return y


def row_deq_mm_T(x: torch.Tensor, w_t: sbvr, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`x @ W.T + bias` for a weight encoded transposed (`sbvr(W, trans=True)` in the reference, sbvr/core.py:244-245:
    `w_t` holds W^T, so `w_t.decode()` is [K, N]).  What the reference's `_sbvr_row_deq_mm_T` call sites compute
    (test_sbvr.py:588-592); the result has the padded width `w_t.in_features_padded`, as there."""
    from . import sbvr_cuda
    if w_t.coeff_idx is None:
        raise ValueError(_r_str("the transposed layout needs codebook indices (the reference has no direct form)"))
    return sbvr_cuda._sbvr_row_deq_mm_T(x.reshape(-1, x.shape[-1]), w_t.bvr, w_t.coeff_idx, w_t.coeff_cache,
                                        bias if bias is not None else w_t._get_dummy_bias(), 0)


def load(filename, device=None, verbose_level=1, cpu_kernel=False, cpu_kernel_v2=False) -> sbvr:
    """Read a file written by `sbvr.save` here or by the reference (sbvr/core.py:1041-1050)."""
    ser = torch.load(filename)      # `_sbvr_serialized` is allow-listed in the package __init__
    obj = sbvr(sbvr_serialized=ser, verbose_level=verbose_level, device=device, cpu_kernel=cpu_kernel,
               cpu_kernel_v2=cpu_kernel_v2)
    if verbose_level > 0:
        print("Loaded SBVR object from: " + str(filename))
        print(obj.get_sbvr_info())
    return obj
