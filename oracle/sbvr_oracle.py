"""CPU oracle for the SBVR quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the GPU kernels are compared against.  It is never
on a product code path: only the test-suite, the smoke check and the CPU
baseline leg of the benchmark import it.  The product package fails loudly when
its CUDA library is missing; it never falls back to anything in here.

It restates, in numpy, the arithmetic of the reference implementation
(MaverickJune/sbvr-cpu-arm).  Each function cites the reference lines it follows.
Parity is pinned: `tests/golden/` holds packed tensors, `decode()` outputs and
`x @ decode().T` products produced by running the reference's own `sbvr/core.py`
(see `tests/golden/make_golden.py`), and `tests/test_oracle.py` checks every
function here against them bit for bit.

Format recap (reference `sbvr/core.py:724-805`, GPU layout):
  bvr         uint32 [Kp/32, N, S]   bit j of bvr[kw, n, s] = plane s of W[n, 32*kw + j]
  coeff_idx   uint8|uint16 [Kp/G, N] codebook line of group g of row n
  coeff_cache float16 [C, S]         codebook
  W[n, k] = fp16_rn( sum_{s=0..S-1} float(cache[idx[k//G, n], s]) * bit_s[n, k] )
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


# --------------------------------------------------------------------------
# bit packing / unpacking
# --------------------------------------------------------------------------
def sel_to_planes(coeff_sel: np.ndarray, S: int) -> np.ndarray:
    """Selector (0 .. 2^S-1) per element -> S bit-planes, plane 0 = MSB.

    Follows `_dec2bin` (sbvr/core.py:815-818): mask = 2**arange(S-1, -1, -1), so
    plane s holds bit (S-1-s) of the selector, which is the s-th entry of the
    row of `itertools.product([0,1], repeat=S)` that the selector indexes
    (sbvr/core.py:345-351).
    """
    sel = np.asarray(coeff_sel).astype(np.int64)
    shifts = np.arange(S - 1, -1, -1, dtype=np.int64)
    return ((sel[..., None] >> shifts) & 1).astype(np.uint8)


def pack_bvr(coeff_sel: np.ndarray, S: int) -> np.ndarray:
    """Selectors [N, Kp] -> bvr uint32 [Kp/32, N, S] (GPU layout).

    Follows `_change_coeff_sel_to_bvr` (sbvr/core.py:842-876): the row-major
    flattened tensor is cut in runs of 32 elements, element e of a run becomes
    bit e (LSB first) of one uint32 per plane; then the view/permute of
    sbvr/core.py:726-730 and :783 turns [S, N, Kp/32] into [Kp/32, N, S].
    """
    sel = np.asarray(coeff_sel)
    N, Kp = sel.shape
    assert Kp % 32 == 0
    planes = sel_to_planes(sel, S)                       # [N, Kp, S]
    planes = planes.reshape(N, Kp // 32, 32, S).astype(np.uint64)
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64)).reshape(1, 1, 32, 1)
    words = (planes * weights).sum(axis=2).astype(np.uint32)   # [N, Kp/32, S]
    return np.ascontiguousarray(words.transpose(1, 0, 2))      # [Kp/32, N, S]


def unpack_bvr(bvr: np.ndarray) -> np.ndarray:
    """bvr uint32 [Kp/32, N, S] -> bits uint8 [N, Kp, S].

    Follows `_change_bvr_to_coeff_sel` (sbvr/core.py:879-901) up to, but not
    including, the recombination into a selector: bit j of word kw is element
    32*kw + j of the row.
    """
    bvr = np.asarray(bvr, dtype=np.uint32)
    KW, N, S = bvr.shape
    shifts = np.arange(32, dtype=np.uint32).reshape(1, 1, 1, 32)
    bits = ((bvr[..., None] >> shifts) & np.uint32(1)).astype(np.uint8)  # [KW,N,S,32]
    return np.ascontiguousarray(bits.transpose(1, 0, 3, 2).reshape(N, KW * 32, S))


def planes_to_sel(bits: np.ndarray) -> np.ndarray:
    """bits [..., S] -> selector, plane 0 = MSB (`_bin2dec`, sbvr/core.py:820-822)."""
    S = bits.shape[-1]
    w = (1 << np.arange(S - 1, -1, -1)).astype(np.int64)
    return (bits.astype(np.int64) * w).sum(-1)


# --------------------------------------------------------------------------
# decode and linear
# --------------------------------------------------------------------------
def group_coeffs(coeff_idx: Optional[np.ndarray], coeff: np.ndarray) -> np.ndarray:
    """Per-(group,row) coefficient lines as float16 [Kp/G, N, S].

    codebook form: coeff = coeff_cache [C, S], coeff_idx [Kp/G, N]
                   (the gather `self.coeff_cache[coeff_idx[i]]`, sbvr/core.py:938)
    direct form  : coeff_idx is None, coeff already is [Kp/G, N, S].
    """
    coeff = np.asarray(coeff, dtype=np.float16)
    if coeff_idx is None:
        assert coeff.ndim == 3
        return coeff
    return coeff[np.asarray(coeff_idx).astype(np.int64)]


def decode(bvr, coeff_idx, coeff, G: int = 256, K: Optional[int] = None) -> np.ndarray:
    """Packed tensors -> dense fp16 weight [N, K].

    Follows `sbvr.decode` (sbvr/core.py:926-949): every element is
    `(bin_combs @ coeff_line)[selector]` (sbvr/core.py:365-366, :940-941), a
    half-precision mat-vec whose products are exact (factor 0 or 1) and whose
    sum is carried in fp32 and rounded to fp16 once; padding columns beyond the
    original K are cut (sbvr/core.py:945-947).  The group length is 256 in the
    reference (sbvr/core.py:222); G = 128 is the same arithmetic with a shorter
    group.
    """
    bits = unpack_bvr(bvr)                                # [N, Kp, S]
    N, Kp, S = bits.shape
    assert Kp % G == 0
    c = group_coeffs(coeff_idx, coeff).astype(np.float32)  # [Kp/G, N, S]
    acc = np.zeros((N, Kp), dtype=np.float32)
    for s in range(S):                                     # plane order, fp32 running sum
        cs = np.repeat(c[:, :, s].T, G, axis=1)            # [N, Kp]
        acc = acc + cs * bits[:, :, s].astype(np.float32)
    W = acc.astype(np.float16)
    if K is not None and K != Kp:
        W = W[:, :K]
    return np.ascontiguousarray(W)


def linear_from_dense(x: np.ndarray, W: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
    """y = fp16( x @ W.T (+ bias) ), products summed in fp32.

    This is the product the reference treats as ground truth for its kernels:
    `a.decode() @ b.decode().T + bias` (test_sbvr.py:321) and the dense matmul its
    Llama flow runs after `sbvr_decompress_on_llama` (sbvr_utils/utils_llama.py:147).
    The reference CUDA kernel for fp16 activations likewise starts the fp32
    running sum, adds the bias and converts to half last
    (sbvr/kernels/sbvr_kernel.cu:145-189).
    """
    x32 = np.asarray(x, dtype=np.float16).astype(np.float32)
    y = x32 @ np.asarray(W, dtype=np.float16).astype(np.float32).T
    if bias is not None and np.size(bias) > 0:
        y = y + np.asarray(bias, dtype=np.float16).astype(np.float32)[None, :]
    return y.astype(np.float16)


def linear(x, bvr, coeff_idx, coeff, bias=None, G: int = 256) -> np.ndarray:
    """fp16 activations [M, K] times packed weight -> fp16 [M, N]."""
    K = np.asarray(x).shape[-1]
    W = decode(bvr, coeff_idx, coeff, G=G, K=K)
    return linear_from_dense(x, W, bias)


def linear_f64(x, bvr, coeff_idx, coeff, bias=None, G: int = 256) -> np.ndarray:
    """Same product in float64 (no output rounding): separates kernel error from
    the fp16 rounding of the reference product (`f64_matmul`, test_sbvr.py:167-170)."""
    K = np.asarray(x).shape[-1]
    W = decode(bvr, coeff_idx, coeff, G=G, K=K).astype(np.float64)
    y = np.asarray(x, dtype=np.float16).astype(np.float64) @ W.T
    if bias is not None and np.size(bias) > 0:
        y = y + np.asarray(bias, dtype=np.float16).astype(np.float64)[None, :]
    return y


# --------------------------------------------------------------------------
# SBVR x SBVR (both operands encoded)
# --------------------------------------------------------------------------
def popc_mm_f64(l_bvr, l_idx, l_coeff, r_bvr, r_idx, r_coeff, bias=None) -> np.ndarray:
    """y[m, n] = sum_g sum_{a,b} popc(l_a & r_b) c^l_a c^r_b (+ bias) in float64, group length 256.

    The quantity `cuda_1xtN_sbvr_mm_T` / `simd_kernel_1xN_popc_first` of the reference compute
    (sbvr/kernels/sbvr_kernel.cu:464-562, sbvr/kernels/sbvr_kernel.cpp:251-399) -- with exact popcounts
    (the reference's 8-bit counters wrap at 256) and no half-precision products.  popc(l_a & r_b) over a group
    is the inner product of the two 0/1 bit vectors, so the sum over planes and groups is the product of the two
    operands decoded WITHOUT rounding: that is how it is formed here.
    """
    def exact(bvr, idx, coeff):
        bits = unpack_bvr(bvr).astype(np.float64)                  # [R, K, S]
        c = group_coeffs(idx, coeff).astype(np.float64)            # [K/256, R, S]
        R, K, S = bits.shape
        cs = np.repeat(c.transpose(1, 0, 2), 256, axis=1)          # [R, K, S]
        return (bits * cs).sum(-1)                                 # [R, K]
    y = exact(l_bvr, l_idx, l_coeff) @ exact(r_bvr, r_idx, r_coeff).T
    if bias is not None and np.size(bias) > 0:
        y = y + np.asarray(bias, dtype=np.float16).astype(np.float64)[None, :]
    return y


# --------------------------------------------------------------------------
# transposed ("row-dequant") weight encoding
# --------------------------------------------------------------------------
def linear_t_f64(x, bvr_t, coeff_idx, coeff, bias=None, G: int = 256, rounded: bool = False) -> np.ndarray:
    """y = x @ W^T (+ bias) in float64 for a weight encoded TRANSPOSED (`sbvr(W, trans=True)`, sbvr/core.py:244-245):
    the packed tensors describe the matrix W^T [K, N], i.e. bvr_t uint32 [N/32, K, S], coeff_idx [N/G, K].

    `cuda_row_deq_mm_T` (sbvr/kernels/sbvr_kernel.cu:121-191) multiplies the activation by the fp32 sum of the selected
    coefficients, NOT rounded to fp16 (`rounded=False`, the default here); `x @ w_t.decode()` is the same product with
    every element rounded to fp16 first (`rounded=True`), the comparator the reference's scripts use for their kernels
    (test_sbvr.py:321-325)."""
    if rounded:
        Wt = decode(bvr_t, coeff_idx, coeff, G=G).astype(np.float64)          # [K, N]
    else:
        bits = unpack_bvr(bvr_t).astype(np.float64)                            # [K, N, S]
        c = group_coeffs(coeff_idx, coeff).astype(np.float64)                  # [N/G, K, S]
        Wt = (bits * np.repeat(c.transpose(1, 0, 2), G, axis=1)).sum(-1)       # [K, N]
    y = np.asarray(x, dtype=np.float16).astype(np.float64) @ Wt
    if bias is not None and np.size(bias) > 0:
        y = y + np.asarray(bias, dtype=np.float16).astype(np.float64)[None, :]
    return y


def max_rel_err(y, ref) -> float:
    """The tolerance metric of the parity tests: max|y - ref| / max|ref|."""
    y = np.asarray(y).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


# --------------------------------------------------------------------------
# seeded synthetic packed weights (stand-in for the slow reference encoder)
# --------------------------------------------------------------------------
def make_packed(N: int, K: int, S: int, G: int = 256, mode: str = "u16", C: Optional[int] = None,
                seed: int = 7, coeff_std: float = 0.01):
    """Bernoulli(0.5) bit-planes in the reference layout, N(0, coeff_std) coefficients.

    mode: "u8" (C <= 256 codebook lines), "u16" (C <= 65536), "direct" (no codebook,
    one coefficient line per (group,row)).  Codebook lines are sorted by |c|
    ascending like the encoder's search space (sbvr/core.py:480-481).
    Returns dict(bvr, coeff_idx, coeff, S, G, N, K, mode).
    """
    assert K % G == 0 and G % 32 == 0
    rng = np.random.default_rng(seed)
    bvr = rng.integers(0, 2**32, size=(K // 32, N, S), dtype=np.uint64).astype(np.uint32)
    if mode == "direct":
        coeff = (rng.standard_normal((K // G, N, S)) * coeff_std).astype(np.float16)
        idx = None
    else:
        if C is None:
            C = 256 if mode == "u8" else 4096
        assert (mode == "u8" and C <= 256) or (mode == "u16" and 256 < C <= 65536)
        cache = rng.standard_normal((C, S)) * coeff_std
        order = np.argsort(np.abs(cache), axis=1)
        cache = np.take_along_axis(cache, order, axis=1)
        coeff = cache.astype(np.float16)
        idx = rng.integers(0, C, size=(K // G, N)).astype(np.uint8 if mode == "u8" else np.uint16)
    return dict(bvr=bvr, coeff_idx=idx, coeff=coeff, S=S, G=G, N=N, K=K, mode=mode)


# --------------------------------------------------------------------------
# C restatement (threaded), used for large sizes and as the timed CPU baseline
# --------------------------------------------------------------------------
_LIB = None


def build_c(force: bool = False) -> str:
    """Compile oracle/sbvr_oracle.c into oracle/libsbvr_oracle.so (gcc, OpenMP)."""
    so = os.path.join(HERE, "libsbvr_oracle.so")
    src = os.path.join(HERE, "sbvr_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", HERE, "libsbvr_oracle.so"])
    return so


def c_lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(HERE, "libsbvr_oracle.so")
        if not os.path.exists(so):
            build_c()
        lib = ctypes.CDLL(so)
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.sbvr_oracle_decode.argtypes = [vp, vp, i, vp, vp, i, i, i, i, i]
        lib.sbvr_oracle_decode.restype = i
        lib.sbvr_oracle_linear.argtypes = [vp, vp, vp, i, vp, vp, vp, i, i, i, i, i, i]
        lib.sbvr_oracle_linear.restype = i
        lib.sbvr_oracle_threads.restype = i
        _LIB = lib
    return _LIB


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _idx_bytes(coeff_idx):
    if coeff_idx is None:
        return 0
    return np.asarray(coeff_idx).dtype.itemsize


def decode_c(bvr, coeff_idx, coeff, G=256, threads=0) -> np.ndarray:
    bvr = np.ascontiguousarray(bvr, dtype=np.uint32)
    KW, N, S = bvr.shape
    coeff = np.ascontiguousarray(coeff, dtype=np.float16)
    idx = None if coeff_idx is None else np.ascontiguousarray(coeff_idx)
    W = np.empty((N, KW * 32), dtype=np.float16)
    rc = c_lib().sbvr_oracle_decode(_ptr(bvr), _ptr(idx), _idx_bytes(idx), _ptr(coeff), _ptr(W),
                                    N, KW * 32, S, G, threads)
    assert rc == 0, rc
    return W


def linear_c(x, bvr, coeff_idx, coeff, bias=None, G=256, threads=0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float16)
    M, K = x.shape
    bvr = np.ascontiguousarray(bvr, dtype=np.uint32)
    KW, N, S = bvr.shape
    assert KW * 32 == K
    coeff = np.ascontiguousarray(coeff, dtype=np.float16)
    idx = None if coeff_idx is None else np.ascontiguousarray(coeff_idx)
    b = None if bias is None or np.size(bias) == 0 else np.ascontiguousarray(bias, dtype=np.float16)
    y = np.empty((M, N), dtype=np.float16)
    rc = c_lib().sbvr_oracle_linear(_ptr(x), _ptr(bvr), _ptr(idx), _idx_bytes(idx), _ptr(coeff), _ptr(b),
                                    _ptr(y), M, N, K, S, G, threads)
    assert rc == 0, rc
    return y
