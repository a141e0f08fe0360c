"""The oracles of the transposed-layout product and of the popcount product, and this library's kernels for them, against
the REFERENCE's own CUDA kernels run on this GPU (oracle/_ref/libsbvr_ref_cuda.so: sbvr/kernels/sbvr_kernel.cu compiled
unchanged for sm_100 behind a C shim).  Skipped where that library has not been built.

Shapes keep to what the reference kernels index safely: N a multiple of 256, K a multiple of 256, even plane counts; the
reference's 4-plane row-dequant kernel (sbvr_kernel.cu:284-359) computes a single activation row, its popcount kernel
(:464-562) counts in 8 bits per 256-bit group (no overflow for random planes) and multiplies coefficients in half2.
"""
import numpy as np
import pytest
import torch

from oracle import ref_cuda
from oracle import sbvr_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available() or ref_cuda.lib() is None,
                                                  reason="reference CUDA kernels not built (make -C oracle ref REF=...)")]


def _dev(p):
    bvr = torch.from_numpy(p["bvr"].view(np.int32)).cuda()
    idx = p["coeff_idx"]
    idx = torch.from_numpy(idx if idx.dtype == np.uint8 else idx.view(np.int16)).cuda()
    return bvr, idx, torch.from_numpy(p["coeff"]).cuda()


@pytest.mark.parametrize("S,M,mode", [(4, 1, "u8"), (4, 1, "u16"), (2, 1, "u16"), (2, 3, "u8")])
def test_transposed_layout_oracle_and_kernel_match_reference_kernel(S, M, mode):
    import sbvr
    N, K = 512, 1024
    p = O.make_packed(K, N, S, G=256, mode=mode, seed=40 + S + M)          # packed W^T: [N/32, K, S], indices [N/256, K]
    bvr, idx, cache = _dev(p)
    rng = np.random.default_rng(S * 10 + M)
    x = rng.standard_normal((M, K)).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float16)
    xt, bt = torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda()
    y_ref = ref_cuda.row_deq_mm_T(xt, bvr, idx, cache, bt, use_shfl=0).cpu().numpy().astype(np.float64)
    oracle = O.linear_t_f64(x, p["bvr"], p["coeff_idx"], p["coeff"], bias)
    assert np.abs(y_ref - oracle).max() / np.abs(oracle).max() <= 2e-3          # the oracle restates the reference kernel
    w_t = sbvr.sbvr.from_packed(bvr, idx if mode == "u8" else idx.view(torch.uint16), cache, group_len=256, device="cuda")
    y = sbvr.row_deq_mm_T(xt, w_t, bt).cpu().numpy().astype(np.float64)
    assert np.abs(y - y_ref).max() / np.abs(y_ref).max() <= 3e-3                # this library's kernel against the reference's


@pytest.mark.parametrize("LS,RS,M", [(4, 4, 1), (2, 4, 3), (4, 2, 5), (2, 2, 8)])
def test_popcount_oracle_and_kernel_match_reference_kernel(LS, RS, M):
    import sbvr
    N, K = 256, 1024
    pl = O.make_packed(M, K, LS, G=256, mode="u8", seed=60 + LS + M)
    pr = O.make_packed(N, K, RS, G=256, mode="u16", C=512, seed=70 + RS)
    lb, li, lc = _dev(pl)
    rb, ri, rc = _dev(pr)
    bias = (np.random.default_rng(M).standard_normal(N) * 0.05).astype(np.float16)
    bt = torch.from_numpy(bias).cuda()
    y_ref = ref_cuda.mm_T(lb, li, lc, rb, ri, rc, bt).cpu().numpy().astype(np.float64)
    oracle = O.popc_mm_f64(pl["bvr"], pl["coeff_idx"], pl["coeff"], pr["bvr"], pr["coeff_idx"], pr["coeff"], bias)
    # the reference multiplies coefficient pairs and popcounts in half2: a few fp16 roundings per term
    assert np.abs(y_ref - oracle).max() / np.abs(oracle).max() <= 1e-2
    a = sbvr.sbvr.from_packed(lb, li, lc, group_len=256, device="cuda")
    b = sbvr.sbvr.from_packed(rb, ri.view(torch.uint16), rc, group_len=256, device="cuda")
    y = sbvr.mm_T(a, b, bt).cpu().numpy().astype(np.float64)
    assert np.abs(y - y_ref).max() / np.abs(y_ref).max() <= 1e-2
