"""The CPU oracle against the golden vectors produced by the reference's own code (no GPU)."""
import numpy as np
import pytest

from oracle import sbvr_oracle as O


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


ALL = ["enc_s2", "enc_s3", "enc_s4", "enc_s4_pad", "syn_u8_s4", "syn_u16_s4", "syn_u8_s2", "syn_u16_s3",
       "syn_u8_s6", "syn_u16_s8"]


@pytest.mark.parametrize("name", ALL)
def test_decode_matches_reference_bit_for_bit(golden, name):
    c = golden[name]
    K = int(c["K"])
    W = O.decode(c["bvr"], c["coeff_idx"], c["coeff_cache"], G=int(c["G"]), K=K)
    assert W.shape == c["decoded"].shape
    assert np.array_equal(_bits(W), _bits(c["decoded"]))


@pytest.mark.parametrize("name", ALL)
def test_c_decode_matches_reference_bit_for_bit(golden, name):
    c = golden[name]
    K = int(c["K"])
    W = O.decode_c(c["bvr"], c["coeff_idx"], c["coeff_cache"], G=int(c["G"]))[:, :K]
    assert np.array_equal(_bits(W), _bits(c["decoded"]))


@pytest.mark.parametrize("name", ALL)
def test_linear_matches_reference_product(golden, name):
    """The reference product is a torch fp16 CPU matmul; ours accumulates in fp32 and rounds once.
    They agree to fp16 rounding: max relative error far below the 1e-2 parity tolerance."""
    c = golden[name]
    K = int(c["K"])
    x = c["x"]
    Kp = c["bvr"].shape[0] * 32
    xp = np.zeros((x.shape[0], Kp), np.float16)
    xp[:, :K] = x
    y = O.linear(xp, c["bvr"], c["coeff_idx"], c["coeff_cache"], bias=c["bias"], G=int(c["G"]))
    assert O.max_rel_err(y, c["y"]) < 2e-3
    yc = O.linear_c(xp, c["bvr"], c["coeff_idx"], c["coeff_cache"], bias=c["bias"], G=int(c["G"]))
    assert O.max_rel_err(yc, c["y"]) < 2e-3
    if "y_nobias" in c:
        y0 = O.linear(xp, c["bvr"], c["coeff_idx"], c["coeff_cache"], G=int(c["G"]))
        assert O.max_rel_err(y0, c["y_nobias"]) < 2e-3


def test_encoder_cases_reproduce_packing(golden):
    """pack_bvr(selectors) must rebuild the reference encoder's bvr tensor exactly: recover the selectors
    from the golden planes, repack, compare."""
    for name in ["enc_s2", "enc_s3", "enc_s4", "enc_s4_pad"]:
        c = golden[name]
        S = int(c["S"])
        bits = O.unpack_bvr(c["bvr"])
        sel = O.planes_to_sel(bits)
        again = O.pack_bvr(sel, S)
        assert again.dtype == np.uint32 and np.array_equal(again, c["bvr"])
        # padding columns of the encoder decode to exactly the value of an all-zero input group element
        assert bits.shape[1] % 256 == 0


def test_padding_is_cut(golden):
    c = golden["enc_s4_pad"]
    assert c["decoded"].shape == (6, 300)
    assert c["bvr"].shape[0] * 32 == 512


@pytest.mark.parametrize("S,G,mode", [(2, 256, "u8"), (3, 256, "u16"), (4, 256, "u16"), (4, 128, "direct"),
                                      (3, 128, "u8"), (2, 128, "direct"), (5, 256, "u8"), (8, 64, "direct")])
def test_c_and_numpy_agree(S, G, mode):
    p = O.make_packed(48, 1024, S, G=G, mode=mode, seed=11 + S)
    W = O.decode(p["bvr"], p["coeff_idx"], p["coeff"], G=G)
    Wc = O.decode_c(p["bvr"], p["coeff_idx"], p["coeff"], G=G)
    assert np.array_equal(_bits(W), _bits(Wc))
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 1024)).astype(np.float16)
    b = (rng.standard_normal(48) * 0.3).astype(np.float16)
    y = O.linear(x, p["bvr"], p["coeff_idx"], p["coeff"], bias=b, G=G)
    yc = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], bias=b, G=G)
    assert O.max_rel_err(yc, y) < 1e-3
    y64 = O.linear_f64(x, p["bvr"], p["coeff_idx"], p["coeff"], bias=b, G=G)
    assert O.max_rel_err(y, y64) < 1e-3


def test_subnormal_coefficients_survive():
    """About 0.5 % of N(0, 0.01) coefficients are fp16 subnormals; decode must keep them exact."""
    p = O.make_packed(8, 256, 2, G=256, mode="u8", C=4, seed=1)
    p["coeff"][:] = np.array([[6e-8, 3e-5], [-6e-8, 5.96e-8], [1e-7, -2e-7], [0, 6.1e-5]], np.float16)
    W = O.decode(p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    Wc = O.decode_c(p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    assert np.array_equal(_bits(W), _bits(Wc))
    assert (np.abs(W.astype(np.float32)) > 0).any()


def test_float_half_roundtrip_tables():
    """The C file's own fp16 conversions against numpy on every bit pattern and on rounding ties."""
    lib = O.c_lib()
    # decode with S=1 and a one-line codebook per value exercises half->float->half on all patterns
    vals = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    finite = vals[np.isfinite(vals)]
    C = 256
    for start in range(0, len(finite), C):
        chunk = finite[start:start + C]
        n = len(chunk)
        bvr = np.full((8, n, 1), 0xFFFFFFFF, np.uint32)
        idx = np.arange(n, dtype=np.uint8).reshape(1, n)
        cache = chunk.reshape(n, 1)
        W = O.decode_c(bvr, idx, cache, G=256)
        expect = (np.float32(0.0) + chunk.astype(np.float32)).astype(np.float16)   # 0 + (-0) = +0
        assert np.array_equal(_bits(W[:, 0]), _bits(expect))
    assert lib.sbvr_oracle_threads() >= 1


def test_popcount_product_oracle_matches_its_definition():
    """`popc_mm_f64` (formed as a product of unrounded decodes) against the popcount sum written out."""
    pl = O.make_packed(3, 512, 4, G=256, mode="u8", seed=1)
    pr = O.make_packed(40, 512, 3, G=256, mode="u16", C=512, seed=2)
    y = O.popc_mm_f64(pl["bvr"], pl["coeff_idx"], pl["coeff"], pr["bvr"], pr["coeff_idx"], pr["coeff"])
    bl, br = O.unpack_bvr(pl["bvr"]), O.unpack_bvr(pr["bvr"])
    cl = O.group_coeffs(pl["coeff_idx"], pl["coeff"]).astype(np.float64)
    cr = O.group_coeffs(pr["coeff_idx"], pr["coeff"]).astype(np.float64)
    for m, n in [(0, 0), (1, 17), (2, 39)]:
        s = 0.0
        for g in range(2):
            for a in range(4):
                for b in range(3):
                    pc = int((bl[m, g * 256:(g + 1) * 256, a] & br[n, g * 256:(g + 1) * 256, b]).sum())
                    s += pc * cl[g, m, a] * cr[g, n, b]
        assert abs(s - y[m, n]) < 1e-12
    dense = O.linear_from_dense(O.decode(pl["bvr"], pl["coeff_idx"], pl["coeff"]),
                                O.decode(pr["bvr"], pr["coeff_idx"], pr["coeff"])).astype(np.float64)
    assert np.abs(y - dense).max() / np.abs(dense).max() < 2e-3


def test_transposed_product_oracle_matches_the_kernel_loop():
    """`linear_t_f64` against a literal loop in the order of the reference kernel for the transposed encoding
    (sbvr/kernels/sbvr_kernel.cu:138-189): word (n/32, k, s), bit n%32, codebook line idx[n/256, k], dot = sum_s c_s * bit_s,
    sum += x * dot.  The rounded variant is x @ decode() of the same packed tensors."""
    N, K, S, M = 256, 24, 3, 2
    p = O.make_packed(K, N, S, G=256, mode="u8", seed=4)               # packed W^T [K rows, N along the bits]
    rng = np.random.default_rng(0)
    x = rng.standard_normal((M, K)).astype(np.float16)
    bias = rng.standard_normal(N).astype(np.float16)
    bvr, idx, cache = p["bvr"], p["coeff_idx"], p["coeff"].astype(np.float64)
    ref = np.zeros((M, N))
    for m in range(M):
        for n in range(N):
            s_ = float(bias[n])
            for k in range(K):
                dot = 0.0
                for s in range(S):
                    bit = (int(bvr[n // 32, k, s]) >> (n % 32)) & 1
                    dot += cache[idx[n // 256, k], s] * bit
                s_ += float(x[m, k]) * dot
            ref[m, n] = s_
    y = O.linear_t_f64(x, bvr, idx, p["coeff"], bias)
    assert np.abs(y - ref).max() <= 1e-12 * max(1.0, np.abs(ref).max())
    Wt = O.decode(bvr, idx, p["coeff"]).astype(np.float64)
    yr = O.linear_t_f64(x, bvr, idx, p["coeff"], bias, rounded=True)
    assert np.allclose(yr, x.astype(np.float64) @ Wt + bias.astype(np.float64)[None, :], rtol=0, atol=1e-12)


@pytest.mark.parametrize("name", ["enc_s2", "enc_s3"])
def test_encoder_restatement_reproduces_the_reference_encoder(golden, name):
    """The sequential encoder walk of oracle/encoder_ref.py, fed with the package's search-space generator (generated on
    the CPU, as the reference run that made the golden vectors did), gives the reference encoder's codebook, indices and
    bit-planes bit for bit."""
    import torch
    from oracle import encoder_ref as E
    from sbvr import encoder
    c = golden[name]
    S = int(c["S"])
    W = torch.from_numpy(c["W"])
    conf = encoder.EncoderConfig(num_sums=S, space_device="cpu")
    r = E.encode(W, S, lambda g, ext: encoder.group_search_space(g, conf, ext))
    N, Kp = W.shape[0], r["Kp"]
    assert np.array_equal(r["lines"].view(np.uint16), c["coeff_cache"].view(np.uint16))
    assert np.array_equal(r["line_of"].reshape(N, Kp // 256).T, c["coeff_idx"].astype(np.int64))
    assert np.array_equal(O.pack_bvr(r["sel"].reshape(N, Kp).astype(np.int64), S), c["bvr"])
