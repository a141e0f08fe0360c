"""Parity of the CUDA kernels with the oracle, through the package API (which calls the C ABI).

decode : bit-exact (integer/fp16 bit patterns equal).
linear : max|y - ref| / max|ref| <= 1e-2 (the tolerance the task states for fp16 outputs), where
         ref is the oracle's fp32-accumulated product of the same inputs; measured errors are
         about 1e-3 (one fp16 rounding of the output) and are asserted tighter where that is stable.
"""
import numpy as np
import pytest
import torch

from oracle import sbvr_oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-2


def to_sbvr(p, device="cuda"):
    import sbvr
    bvr = torch.from_numpy(p["bvr"].view(np.int32))
    idx = p.get("coeff_idx")
    if idx is not None:
        idx = torch.from_numpy(idx) if idx.dtype == np.uint8 else torch.from_numpy(idx.view(np.int16)).view(torch.uint16)
    coeff = torch.from_numpy(p["coeff"] if "coeff" in p else p["coeff_cache"])
    return sbvr.sbvr.from_packed(bvr, idx, coeff, group_len=int(p["G"]), device=torch.device(device))


def h2n(t):
    return t.detach().cpu().numpy()


def check_status():
    from sbvr import _lib
    for (dev, st), ws in _lib._workspaces.items():
        assert ws.status(st) == 0, "a device-side wait timed out"


GOLD = ["enc_s2", "enc_s3", "enc_s4", "enc_s4_pad", "syn_u8_s4", "syn_u16_s4", "syn_u8_s2", "syn_u16_s3",
        "syn_u8_s6", "syn_u16_s8"]


@pytest.mark.parametrize("name", GOLD)
def test_decode_golden_bit_exact(golden, name):
    import sbvr
    c = dict(golden[name])
    c["coeff"] = c["coeff_cache"]
    w = to_sbvr(c)
    w.original_data_shape = torch.Size((int(c["N"]), int(c["K"])))
    W = h2n(w.decode())
    assert W.shape == c["decoded"].shape
    assert np.array_equal(W.view(np.uint16), c["decoded"].view(np.uint16))


@pytest.mark.parametrize("name", GOLD)
@pytest.mark.parametrize("algo", [1, 0])
def test_linear_golden(golden, name, algo):
    """Against the reference's own product `x @ decode().T + bias` stored in the fixtures."""
    import sbvr
    c = dict(golden[name])
    c["coeff"] = c["coeff_cache"]
    w = to_sbvr(c)
    w.original_data_shape = torch.Size((int(c["N"]), int(c["K"])))
    x = torch.from_numpy(c["x"]).cuda()
    b = torch.from_numpy(c["bias"]).cuda()
    y = h2n(sbvr.linear(x, w, b, algo=algo))
    assert O.max_rel_err(y, c["y"]) <= TOL
    assert O.max_rel_err(y, c["y"]) <= 3e-3
    check_status()


@pytest.mark.parametrize("S", [2, 3, 4])
@pytest.mark.parametrize("G", [256, 128])
@pytest.mark.parametrize("mode", ["u8", "u16", "direct"])
def test_decode_bit_exact_grid(S, G, mode):
    p = O.make_packed(192, 1024, S, G=G, mode=mode, seed=S * 10 + G)
    w = to_sbvr(p)
    W = h2n(w.decode())
    ref = O.decode_c(p["bvr"], p["coeff_idx"], p["coeff"], G=G)
    assert np.array_equal(W.view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("S", [2, 3, 4])
@pytest.mark.parametrize("G", [256, 128])
@pytest.mark.parametrize("mode", ["u8", "u16", "direct"])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("algo", [1, 2])
def test_linear_grid(S, G, mode, M, algo):
    import sbvr
    N, K = 320, 1536
    p = O.make_packed(N, K, S, G=G, mode=mode, seed=S * 100 + G + M)
    w = to_sbvr(p)
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float16)
    b = (rng.standard_normal(N) * 0.3).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], bias=b, G=G)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, torch.from_numpy(b).cuda(), algo=algo))
    err = O.max_rel_err(y, ref)
    assert err <= TOL, err
    assert err <= 2e-3, err
    check_status()


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("S", [2, 3, 4])
def test_linear_llama_shapes_m1(shape, S):
    """The four Llama-3-8B layer shapes at M=1, codebook u16, G=256, both kernels against the threaded C oracle."""
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, S, G=256, mode="u16", C=4096, seed=7)
    w = to_sbvr(p)
    rng = np.random.default_rng(1234)
    x = rng.standard_normal((1, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    xt = torch.from_numpy(x).cuda()
    for algo in (2, 1):
        y = h2n(sbvr.linear(xt, w, None, algo=algo))
        err = O.max_rel_err(y, ref)
        assert err <= TOL, (algo, err)
    check_status()


@pytest.mark.parametrize("M", [4, 16, 32])
def test_linear_small_m(M):
    import sbvr
    N, K, S = 1024, 4096, 4
    p = O.make_packed(N, K, S, G=256, mode="u16", C=4096, seed=3)
    w = to_sbvr(p)
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None))
    assert O.max_rel_err(y, ref) <= TOL
    check_status()


@pytest.mark.parametrize("S", [2, 3, 4])
@pytest.mark.parametrize("G,mode", [(256, "u16"), (128, "u8"), (256, "direct")])
@pytest.mark.parametrize("M", [5, 16, 32, 33, 64, 100, 128, 200, 256, 300, 515])
def test_linear_batched_gemm_grid(S, G, mode, M):
    """The tcgen05 GEMM with in-kernel dequantisation (algo 3) against the oracle, every activation tile width,
    ragged M, split K (few tiles) and several work items per CTA."""
    import sbvr
    N, K = 384, 1536
    p = O.make_packed(N, K, S, G=G, mode=mode, seed=S * 1000 + G + M)
    w = to_sbvr(p)
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float16)
    b = (rng.standard_normal(N) * 0.3).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], bias=b, G=G)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, torch.from_numpy(b).cuda(), algo=3))
    err = O.max_rel_err(y, ref)
    assert err <= TOL, err
    assert err <= 3e-3, err
    check_status()


@pytest.mark.parametrize("shape,M", [((4096, 4096), 16), ((1024, 4096), 32), ((4096, 14336), 16), ((14336, 4096), 512)])
def test_linear_batched_gemm_llama_shapes(shape, M):
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, 4, G=256, mode="u16", C=4096, seed=11)
    w = to_sbvr(p)
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    xt = torch.from_numpy(x).cuda()
    y = sbvr.linear(xt, w, None, algo=3)
    err = O.max_rel_err(h2n(y), ref)
    assert err <= TOL, err
    assert torch.equal(y, sbvr.linear(xt, w, None, algo=3))       # split-K sums in a fixed order
    check_status()


def test_linear_is_linear_and_deterministic():
    """Size-independent properties at a full layer shape: y(ax1 + x2) = a y(x1) + y(x2) up to rounding, and
    two calls on the same inputs give identical bits (the split-K reduction order is fixed)."""
    import sbvr
    N, K, S = 4096, 4096, 4
    p = O.make_packed(N, K, S, G=256, mode="u16", C=4096, seed=21)
    w = to_sbvr(p)
    g = torch.Generator(device="cuda").manual_seed(5)
    x1 = torch.randn((1, K), device="cuda", generator=g).half()
    x2 = torch.randn((1, K), device="cuda", generator=g).half()
    y1 = sbvr.linear(x1, w).float()
    y2 = sbvr.linear(x2, w).float()
    y12 = sbvr.linear((2 * x1.float() + x2.float()).half(), w).float()
    scale = y12.abs().max()
    assert ((2 * y1 + y2 - y12).abs().max() / scale).item() < 1e-2
    a = sbvr.linear(x1, w)
    b = sbvr.linear(x1, w)
    assert torch.equal(a, b)
    check_status()


def test_zero_and_extreme_activations():
    import sbvr
    N, K, S = 128, 512, 4
    p = O.make_packed(N, K, S, G=256, mode="u8", seed=2)
    w = to_sbvr(p)
    x = np.zeros((2, K), np.float16)
    x[1, :256] = 60000.0          # near the fp16 maximum in one group
    x[1, 256:] = 6e-8             # subnormals only in the other
    ref = O.linear_f64(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    for algo in (1, 2):
        y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None, algo=algo)).astype(np.float64)
        assert np.all(y[0] == 0)
        ok = np.isfinite(ref[1]) & (np.abs(ref[1]) < 65000)
        assert np.abs(y[1][ok] - ref[1][ok]).max() / np.abs(ref[1][ok]).max() <= TOL
    check_status()


def test_mm_T_with_encoded_lhs(golden):
    """Reference test 'Case 1' (test_sbvr.py:321-325, :351-352): decode(a) @ decode(b).T + bias."""
    import sbvr
    ca, cb = dict(golden["syn_u8_s2"]), dict(golden["syn_u8_s2"])
    ca["coeff"] = ca["coeff_cache"]
    a = to_sbvr(ca)
    b = to_sbvr(ca)
    bias = torch.from_numpy(ca["bias"]).cuda()
    y = h2n(sbvr.mm_T(a, b, bias))
    A = ca["decoded"]
    ref = O.linear_from_dense(A, A, ca["bias"])
    assert O.max_rel_err(y, ref) <= TOL


def test_host_buffer_entry_point():
    """The end-to-end C entry point with host activations and host result."""
    import ctypes
    import sbvr
    from sbvr import _lib
    N, K, S = 1024, 4096, 4
    p = O.make_packed(N, K, S, G=256, mode="u16", C=4096, seed=9)
    w = to_sbvr(p)
    x = torch.randn((1, K)).half().pin_memory()
    y = torch.empty((1, N), dtype=torch.float16).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(0, st)
    b, ix, ib, c, C = w._abi_args()
    rc = _lib.lib.sbvr_linear_f16_host(x.data_ptr(), b, ix, ib, c, C, None, y.data_ptr(), 1, N, K, S, 256, 0,
                                       ws.handle, st)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    ref = O.linear_c(x.numpy(), p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    assert O.max_rel_err(y.numpy(), ref) <= TOL
    check_status()


@pytest.mark.parametrize("K", [256, 512, 768])
@pytest.mark.parametrize("M", [1, 2])
def test_linear_fewer_k_blocks_than_warpgroups(K, M):
    """Row-parallel shards of small models leave a CTA fewer 256-k blocks than it has compute warpgroups."""
    import sbvr
    N, S = 512, 4
    p = O.make_packed(N, K, S, G=256, mode="u8", seed=K + M)
    w = to_sbvr(p)
    rng = np.random.default_rng(K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None, algo=2))
    assert O.max_rel_err(y, ref) <= TOL
    check_status()


@pytest.mark.parametrize("M", [1, 2, 4])
@pytest.mark.parametrize("K", [1024, 3584])
def test_fused_silu_mul_linear_equals_separate_kernels(M, K):
    """SiLU(gate) * up folded into the decode GEMV gives the bits of sbvr_silu_mul_f16 followed by sbvr_linear_f16."""
    import sbvr
    from sbvr import _lib
    from sbvr.core import XOP_SILU_MUL, linear_fused
    N, S = 512, 4
    p = O.make_packed(N, K, S, G=256, mode="u16", C=1024, seed=K + M)
    w = to_sbvr(p)
    g = torch.Generator(device="cuda").manual_seed(M)
    gu = torch.randn((M, 2 * K), device="cuda", generator=g).half()
    act = torch.empty((M, K), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.sbvr_silu_mul_f16(gu.data_ptr(), act.data_ptr(), M, K, st))
    y_sep = sbvr.linear(act, w, None, algo=2)
    y = torch.empty_like(y_sep)
    assert linear_fused(XOP_SILU_MUL, gu, w, y)
    assert torch.equal(y, y_sep)
    ref = O.linear_c(h2n(act), p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    assert O.max_rel_err(h2n(y), ref) <= TOL
    check_status()


@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("with_delta", [True, False])
def test_fused_add_rmsnorm_linear(M, with_delta):
    """Residual add + RMSNorm folded into the decode GEMV: the new residual is exact, the product matches the
    separate kernels (only the fp32 summation order of the mean square differs)."""
    import sbvr
    from sbvr import _lib
    from sbvr.core import XOP_ADD_RMSNORM, linear_fused
    N, K, S = 768, 2048, 4
    p = O.make_packed(N, K, S, G=256, mode="u8", seed=M + 7)
    w = to_sbvr(p)
    g = torch.Generator(device="cuda").manual_seed(3 * M)
    h = torch.randn((M, K), device="cuda", generator=g).half()
    d = torch.randn((M, K), device="cuda", generator=g).half() if with_delta else None
    nw = (1 + 0.2 * torch.randn(K, device="cuda", generator=g)).half()
    st = torch.cuda.current_stream().cuda_stream
    h_sep, xn = torch.empty_like(h), torch.empty_like(h)
    _lib.check(_lib.lib.sbvr_add_rmsnorm_f16(h.data_ptr(), None if d is None else d.data_ptr(), nw.data_ptr(),
                                             h_sep.data_ptr(), xn.data_ptr(), M, K, 1e-5, st))
    y_sep = sbvr.linear(xn, w, None, algo=2)
    y, h_out = torch.empty_like(y_sep), torch.empty_like(h)
    assert linear_fused(XOP_ADD_RMSNORM, h, w, y, delta=d, norm_weight=nw, h_out=h_out, eps=1e-5)
    assert torch.equal(h_out, h_sep)
    assert ((y.float() - y_sep.float()).abs().max() / y_sep.float().abs().max()).item() < 2e-3
    check_status()


@pytest.mark.parametrize("LS,RS", [(2, 2), (4, 4), (3, 4), (4, 2), (2, 3)])
@pytest.mark.parametrize("M", [1, 3, 11])
def test_popcount_mm_T_both_operands_encoded(LS, RS, M):
    """`sbvr.mm_T(lhs_sbvr, rhs_sbvr, bias)` on the popcount kernel against the exact product of the two encodings,
    and against the reference's comparator for this kernel, decode(a) @ decode(b).T + bias (test_sbvr.py:321-325)."""
    import sbvr
    N, K = 328, 1024
    pl = O.make_packed(M, K, LS, G=256, mode="u8", seed=100 + LS * 10 + M)
    pr = O.make_packed(N, K, RS, G=256, mode="u16", C=512, seed=200 + RS)
    a, b = to_sbvr(pl), to_sbvr(pr)
    rng = np.random.default_rng(M)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float16)
    y = h2n(sbvr.mm_T(a, b, torch.from_numpy(bias).cuda())).astype(np.float64)
    ref = O.popc_mm_f64(pl["bvr"], pl["coeff_idx"], pl["coeff"], pr["bvr"], pr["coeff_idx"], pr["coeff"], bias)
    assert np.abs(y - ref).max() / np.abs(ref).max() <= 2e-3
    dense = O.linear_from_dense(O.decode(pl["bvr"], pl["coeff_idx"], pl["coeff"]),
                                O.decode(pr["bvr"], pr["coeff_idx"], pr["coeff"]), bias).astype(np.float64)
    assert np.abs(y - dense).max() / np.abs(dense).max() <= TOL


@pytest.mark.parametrize("shape", [(128256, 4096), (6144, 4096), (28672, 4096), (8192, 8192), (10240, 8192), (8192, 28672)])
def test_linear_model_shapes_m1(shape):
    """The shapes the Llama models actually launch at batch 1: lm_head, fused q|k|v and gate|up of the 8B model, and
    hidden / fused q|k|v / down of the 70B model (many row tiles per CTA, long K)."""
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, 4, G=256, mode="u16", C=4096, seed=N % 97)
    w = to_sbvr(p)
    rng = np.random.default_rng(K)
    x = rng.standard_normal((1, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None, algo=2))
    err = O.max_rel_err(y, ref)
    assert err <= TOL, err
    assert err <= 2e-3, err
    check_status()


@pytest.mark.parametrize("S", [2, 3, 4])
@pytest.mark.parametrize("mode", ["u8", "u16"])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 7])
def test_row_deq_mm_T_transposed_encoding(S, mode, M):
    """`sbvr.sbvr_cuda._sbvr_row_deq_mm_T(x, bvr, idx, cache, bias, use_shfl)` on the transposed encoding (groups of 256
    along the OUTPUT dimension) against the reference kernel's arithmetic (unrounded dequantised elements) and against
    x @ w_t.decode() + bias, the comparator of the reference's scripts.  K = 800 is not a multiple of the block's 256."""
    import sbvr
    N, K = 512, 800
    p = O.make_packed(K, N, S, G=256, mode=mode, seed=300 + S)          # packed W^T: K rows, N along the bits
    w_t = to_sbvr(p)
    rng = np.random.default_rng(7 * M + S)
    x = rng.standard_normal((M, K)).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float16)
    y = h2n(sbvr.sbvr_cuda._sbvr_row_deq_mm_T(torch.from_numpy(x).cuda(), w_t.bvr, w_t.coeff_idx, w_t.coeff_cache,
                                              torch.from_numpy(bias).cuda(), 0)).astype(np.float64)
    ref = O.linear_t_f64(x, p["bvr"], p["coeff_idx"], p["coeff"], bias)
    assert y.shape == (M, N)
    assert np.abs(y - ref).max() / np.abs(ref).max() <= 2e-3
    dec = O.linear_t_f64(x, p["bvr"], p["coeff_idx"], p["coeff"], bias, rounded=True)
    assert np.abs(y - dec).max() / np.abs(dec).max() <= TOL
    # no bias = a tensor whose length is not N; the wrapper on the container gives the same numbers
    y0 = sbvr.row_deq_mm_T(torch.from_numpy(x).cuda(), w_t)
    y1 = sbvr.sbvr_cuda._sbvr_row_deq_mm_T(torch.from_numpy(x).cuda(), w_t.bvr, w_t.coeff_idx, w_t.coeff_cache,
                                           w_t._get_dummy_bias(), 1)
    assert torch.equal(y0, y1)
    ref0 = O.linear_t_f64(x, p["bvr"], p["coeff_idx"], p["coeff"])
    assert np.abs(h2n(y0).astype(np.float64) - ref0).max() / np.abs(ref0).max() <= 2e-3
    check_status()


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_row_deq_mm_T_llama_shapes_deterministic(shape):
    """Layer shapes (N x K) of Llama-3-8B at M = 1: the decoded transposed weight is the transpose of a decoded plain one,
    so the product must agree with `x @ decode().T` computed on the GPU; K is split over blocks here, and two runs give
    the same bits."""
    import sbvr
    N, K = shape
    p = O.make_packed(K, N, 4, G=256, mode="u16", C=4096, seed=11)
    w_t = to_sbvr(p)
    x = torch.randn(1, K, dtype=torch.float16, device="cuda", generator=torch.Generator("cuda").manual_seed(5))
    y = sbvr.row_deq_mm_T(x, w_t)
    ref = x.double() @ w_t.decode().double()
    assert ((y.double() - ref).abs().max() / ref.abs().max()).item() <= 2e-3
    assert torch.equal(y, sbvr.row_deq_mm_T(x, w_t))
    check_status()


@pytest.mark.parametrize("shape", [(14336, 4096), (4096, 14336)])
def test_prefill_gemm_m2048_llama_shapes(shape):
    """The prefill configuration itself: M = 2048 tokens on the gate/up and down shapes, against the dense fp32 product of
    the decoded weight (the CPU oracle decodes, the comparison product runs on the GPU in fp32)."""
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, 4, G=256, mode="u16", C=4096, seed=N % 89)
    w = to_sbvr(p)
    g = torch.Generator(device="cuda").manual_seed(K)
    x = torch.randn((2048, K), device="cuda", generator=g).half()
    Wd = torch.from_numpy(O.decode_c(p["bvr"], p["coeff_idx"], p["coeff"], G=256)).cuda()
    ref = (x.float() @ Wd.float().T)
    y = sbvr.linear(x, w, None).float()
    err = ((y - ref).abs().max() / ref.abs().max()).item()
    assert err <= TOL, err
    assert err <= 3e-3, err
    check_status()


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_group128_direct_llama_shapes(shape, M):
    """Group length 128 with one coefficient line per (group, row) (no codebook: 128 k groups x 14336 rows exceed 65536
    lines) on the four Llama-3-8B shapes."""
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, 4, G=128, mode="direct", seed=N % 83 + M)
    w = to_sbvr(p)
    rng = np.random.default_rng(M + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=128)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None))
    err = O.max_rel_err(y, ref)
    assert err <= TOL, err
    assert err <= 3e-3, err
    check_status()


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [16, 32])
@pytest.mark.parametrize("S", [2, 3, 4])
def test_small_batches_llama_shapes(shape, M, S):
    """The small-batch corners of the sweep configuration: M in {16, 32} x bit-plane counts {2, 3, 4} on every layer shape."""
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, S, G=256, mode="u16", C=4096, seed=S * 7 + M)
    w = to_sbvr(p)
    rng = np.random.default_rng(M * S)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None))
    err = O.max_rel_err(y, ref)
    assert err <= TOL, err
    assert err <= 3e-3, err
    check_status()


@pytest.mark.parametrize("S", [2, 3, 4])
@pytest.mark.parametrize("G,mode", [(256, "u16"), (128, "u8"), (256, "direct"), (128, "direct")])
@pytest.mark.parametrize("M", [2, 5, 8, 15, 16, 17, 24, 31, 32])
def test_linear_small_batch_kernel_grid(S, G, mode, M):
    """The small-batch tensor-core kernel (algo 4) against the oracle: both digit packings (M <= 16 and M > 16), ragged M,
    every plane count and coefficient form, few tiles (k blocks of a tile group spread over CTAs) and a ragged tile group."""
    import sbvr
    if G == 128 and M > 16:
        pytest.skip("two groups per 256-k block: up to 16 activation rows on this kernel")
    N, K = 320, 1536
    p = O.make_packed(N, K, S, G=G, mode=mode, seed=S * 1000 + G + M)
    w = to_sbvr(p)
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float16)
    x[:, ::5] *= 16.0                                   # a few large activations per block: small ones keep their low bits
    b = (rng.standard_normal(N) * 0.3).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], bias=b, G=G)
    xt, bt = torch.from_numpy(x).cuda(), torch.from_numpy(b).cuda()
    y = sbvr.linear(xt, w, bt, algo=4)
    err = O.max_rel_err(h2n(y), ref)
    assert err <= TOL, err
    assert err <= 3e-3, err
    assert torch.equal(y, sbvr.linear(xt, w, bt, algo=4))          # fixed summation order: the same bits on every run
    check_status()


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [5, 16, 32])
def test_linear_small_batch_kernel_llama_shapes(shape, M):
    """Algo 4 on the four layer shapes."""
    import sbvr
    N, K = shape
    p = O.make_packed(N, K, 4, G=256, mode="u16", C=4096, seed=M + N // 1024)
    w = to_sbvr(p)
    rng = np.random.default_rng(M + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    xt = torch.from_numpy(x).cuda()
    y = sbvr.linear(xt, w, None, algo=4)
    err = O.max_rel_err(h2n(y), ref)
    assert err <= TOL, err
    assert err <= 3e-3, err
    check_status()


def test_small_batch_kernel_non_finite_row_poisons_only_that_row():
    import sbvr
    N, K, M = 256, 1024, 6
    p = O.make_packed(N, K, 4, G=256, mode="u16", C=4096, seed=77)
    w = to_sbvr(p)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((M, K)).astype(np.float16)
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    x[2, 700] = np.inf
    y = h2n(sbvr.linear(torch.from_numpy(x).cuda(), w, None, algo=4))
    assert np.isnan(y[2]).all()
    keep = [0, 1, 3, 4, 5]
    assert O.max_rel_err(y[keep], ref[keep]) <= TOL
    check_status()
