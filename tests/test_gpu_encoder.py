"""The GPU encoder (`sbvr.sbvr(data, encoder_config)`, sbvr/encoder.py + csrc/encode.cu) against the reference encoder's
golden output and against the CPU restatement of its error function (oracle/encoder_ref.py)."""
import numpy as np
import pytest
import torch

from oracle import encoder_ref as E
from oracle import sbvr_oracle as O

pytestmark = pytest.mark.gpu


def _u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.uint16 else t.cpu().numpy()


@pytest.mark.parametrize("S", [1, 2, 3, 4])
def test_error_function_and_selectors_match_the_restatement(S):
    """`sbvr_encode_mse_f16` / `sbvr_encode_select_f16` on seeded groups and lines: the fp16 steps are the reference's, so
    the selectors are identical and the MSEs differ only by the order of the fp32 sum over the 256 values."""
    from sbvr import encoder
    g = torch.Generator().manual_seed(S)
    data = (torch.randn((5, 256), generator=g) * 0.02).half()
    lines = (torch.randn((777, S), generator=g) * 0.02).half()
    ref = E.mse_table(data, lines)
    got = encoder._mse(data.cuda(), lines.cuda(), S).cpu().numpy()
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= 2e-6 * ref.max()
    which = torch.tensor([0, 5, 776, 13, 400], dtype=torch.int32)
    sel = torch.empty((5, 256), dtype=torch.uint8, device="cuda")
    encoder._select(data.cuda(), lines.cuda(), which.cuda(), S, sel)
    for b in range(5):
        assert np.array_equal(sel[b].cpu().numpy(), E.selectors(data[b], lines[int(which[b])]))


@pytest.mark.parametrize("S", [2, 3, 4])
def test_pack_selectors_is_the_reference_layout(S):
    from sbvr import encoder
    rng = np.random.default_rng(S)
    sel = rng.integers(0, 2 ** S, size=(7, 512), dtype=np.uint8)
    bvr = encoder.pack_selectors(torch.from_numpy(sel).cuda(), S)
    assert np.array_equal(bvr.cpu().view(torch.int32).numpy().view(np.uint32), O.pack_bvr(sel.astype(np.int64), S))


@pytest.mark.parametrize("name", ["enc_s2", "enc_s3", "enc_s4", "enc_s4_pad"])
def test_encoder_reproduces_the_reference_encoder(golden, name):
    """Same input as the golden case, search spaces generated on the CPU like the reference run that made it: the
    codebook, the indices and the bit-planes are the reference's, bit for bit; and `decode()` gives its decoded weight."""
    import sbvr
    c = golden[name]
    S = int(c["S"])
    W = torch.from_numpy(c["W"])
    w = sbvr.sbvr(W, encoder_config={"num_sums": S, "space_device": "cpu"}, verbose_level=0)
    assert np.array_equal(_u16(w.coeff_cache).view(np.uint16), c["coeff_cache"].view(np.uint16))
    assert np.array_equal(_u16(w.coeff_idx), c["coeff_idx"])
    assert np.array_equal(w.bvr.cpu().view(torch.int32).numpy().view(np.uint32), c["bvr"])
    assert np.array_equal(w.decode().cpu().numpy().view(np.uint16), c["decoded"].view(np.uint16))


def _mse_of(w, W):
    return float(((w.decode().float().cpu() - W.float()) ** 2).mean())


@pytest.mark.parametrize("name", ["enc_s2", "enc_s4", "enc_s4_pad"])
def test_encoder_with_gpu_generated_search_space_is_as_good(golden, name):
    """Search spaces generated on the GPU (the default; what the reference does when it has a GPU): candidates may differ
    from a CPU run in the last fp16 bit, the quality must not."""
    import sbvr
    c = golden[name]
    W = torch.from_numpy(c["W"])
    w = sbvr.sbvr(W, encoder_config={"num_sums": int(c["S"])}, verbose_level=0)
    ref_mse = float(((torch.from_numpy(c["decoded"]).float() - W.float()) ** 2).mean())
    assert _mse_of(w, W) <= 1.02 * ref_mse
    assert tuple(w.decode().shape) == tuple(W.shape)


def test_batched_lookup_equals_the_sequential_walk():
    """The speculative batch (codebook look-up of many groups in one launch, one-line updates after each addition) must
    decide exactly as a walk that looks up one group at a time; trans=True encodes the transpose."""
    import sbvr
    g = torch.Generator().manual_seed(3)
    W = (torch.randn((48, 512), generator=g) * 0.02).half()
    W[:, :256] *= torch.linspace(0.5, 3.0, 48).view(-1, 1).half()         # spread the statistics: more misses
    a = sbvr.sbvr(W, encoder_config={"num_sums": 3, "batch_groups": 1}, verbose_level=0)
    b = sbvr.sbvr(W, encoder_config={"num_sums": 3, "batch_groups": 37}, verbose_level=0)
    assert torch.equal(a.coeff_cache, b.coeff_cache)
    assert torch.equal(a.coeff_idx.view(torch.uint8), b.coeff_idx.view(torch.uint8))
    assert torch.equal(a.bvr.view(torch.int32), b.bvr.view(torch.int32))
    assert a.encoder_stats == b.encoder_stats and a.encoder_stats["cache_hits"] > 0
    t = sbvr.sbvr(W[:, :256].contiguous(), encoder_config={"num_sums": 2}, verbose_level=0, trans=True)
    assert tuple(t.bvr.shape) == (8, 256, 2)                               # W^T is [256, 48], padded to 256 along the bits
    assert tuple(t.decode().shape) == (256, 48)


def test_encode_then_linear_end_to_end():
    """A really encoded weight (not synthetic planes) through the decode GEMV and the batched GEMM: the product with the
    packed weight equals x @ decode().T within the fp16 tolerance, and stays close to the product with the dense weight."""
    import sbvr
    g = torch.Generator().manual_seed(42)
    W = (torch.randn((1024, 4096), generator=g) * 0.02).half().cuda()
    w = sbvr.sbvr(W, encoder_config={"num_sums": 4}, verbose_level=0)
    Wd = w.decode()
    assert float(((Wd.float() - W.float()) ** 2).mean() / (W.float() ** 2).mean()) < 0.02
    for M in (1, 16):
        x = torch.randn((M, 4096), generator=g).half().cuda()
        y = sbvr.linear(x, w).double()
        ref = x.double() @ Wd.double().T
        assert float((y - ref).abs().max() / ref.abs().max()) <= 1e-2
        dense = x.double() @ W.double().T
        assert float((y - dense).abs().max() / dense.abs().max()) < 0.2
