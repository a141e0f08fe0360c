"""The allocation-free entry point `sbvr_linear_f16_noalloc`, called through the C ABI.

It exists for callers that are forbidden to allocate device memory (a serving process that owns the whole GPU
arena, a latency-critical loop, code next to an open stream capture): it takes no workspace and keeps its scratch
in a fixed 4 MiB array inside the library.  The tests check that it gives the same result as the regular entry point
`sbvr_linear_f16` and as the CPU oracle, on two calls in a row (the second call meets whatever the first left in the
shared array) with a different problem in between, that the device's free memory does not move while it is called,
that a batch whose scratch fits is served by the batched kernel, and that one whose scratch cannot fit is refused
before anything is launched.

The file name sorts last so that a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from oracle import sbvr_oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-2          # same tolerance as tests/test_gpu_parity.py: max|a - b| / max|b|


def _packed(N, K, S, C, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    bvr = torch.randint(-2**31, 2**31 - 1, (K // 32, N, S), dtype=torch.int32, device=dev, generator=g)
    idx = torch.randint(0, C, (K // 256, N), device=dev, generator=g)
    idx = idx.to(torch.uint8) if C <= 256 else idx.to(torch.int16)
    cache = (torch.randn((C, S), device=dev, generator=g) * 0.01).half()
    return bvr, idx, cache


def _oracle(x, w, bias=None):
    """x @ decode(w).T + bias by the CPU oracle (threaded C restatement of the reference arithmetic)."""
    bvr, idx, cache = w
    bvr_n = bvr.cpu().numpy().view(np.uint32)
    idx_n = idx.cpu().numpy()
    idx_n = idx_n if idx_n.dtype == np.uint8 else idx_n.view(np.uint16)
    b = None if bias is None else bias.cpu().numpy()
    return torch.from_numpy(O.linear_c(x.cpu().numpy(), bvr_n, idx_n, cache.cpu().numpy(), bias=b, G=256))


def _max_rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def _call_noalloc(L, x, w, y, M, N, K, S, C, bias=None):
    bvr, idx, cache = w
    st = torch.cuda.current_stream().cuda_stream
    return L.sbvr_linear_f16_noalloc(x.data_ptr(), bvr.data_ptr(), idx.data_ptr(), idx.element_size(), cache.data_ptr(),
                                     C, None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K, S, 256, st)


def _call_regular(_lib, x, w, y, M, N, K, S, C, bias=None):
    bvr, idx, cache = w
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(torch.cuda.current_device(), st, _lib.workspace_bytes(torch.cuda.current_device(), M, N, K))
    return _lib.lib.sbvr_linear_f16(x.data_ptr(), bvr.data_ptr(), idx.data_ptr(), idx.element_size(), cache.data_ptr(),
                                    C, None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K, S, 256, 0,
                                    ws.handle, st)


@pytest.mark.parametrize("M", [1, 3])
def test_noalloc_matches_regular_entry_point_twice(M):
    import sbvr  # noqa: F401
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    N, K, S, C = 4096, 4096, 4, 4096
    w = _packed(N, K, S, C, 11, dev)
    x = torch.randn((M, K), device=dev).half()
    bias = (torch.randn((N,), device=dev) * 0.3).half()
    y_ref = torch.empty((M, N), dtype=torch.float16, device=dev)
    assert _call_regular(_lib, x, w, y_ref, M, N, K, S, C, bias) == 0
    # a second, different problem that is run between the two calls and dirties the shared scratch
    N2, K2 = 1024, 1536
    w2 = _packed(N2, K2, 3, 200, 12, dev)
    x2 = torch.randn((2, K2), device=dev).half()
    y2_ref = torch.empty((2, N2), dtype=torch.float16, device=dev)
    assert _call_regular(_lib, x2, w2, y2_ref, 2, N2, K2, 3, 200) == 0
    y_or = _oracle(x, w, bias)

    # every buffer exists before the calls; one warm-up call does the per-device and per-kernel set-up
    outs = [torch.full((M, N), float("nan"), dtype=torch.float16, device=dev) for _ in range(2)]
    y2 = torch.full((2, N2), float("nan"), dtype=torch.float16, device=dev)
    warm = torch.empty((M, N), dtype=torch.float16, device=dev)
    assert _call_noalloc(L, x, w, warm, M, N, K, S, C, bias) == 0
    assert _call_noalloc(L, x2, w2, y2, 2, N2, K2, 3, 200) == 0
    torch.cuda.synchronize()
    y2.fill_(float("nan"))
    free_before, _ = torch.cuda.mem_get_info()      # the driver's view: a cudaMalloc inside the library would show here
    for call in range(2):
        rc = _call_noalloc(L, x, w, outs[call], M, N, K, S, C, bias)
        assert rc == 0, _lib.strerror(rc)
        if call == 0:
            rc = _call_noalloc(L, x2, w2, y2, 2, N2, K2, 3, 200)
            assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before, (free_before, free_after)
    assert _max_rel(y2, y2_ref) <= TOL
    for y in outs:
        assert torch.isfinite(y).all()
        assert _max_rel(y, y_ref) <= TOL            # the existing entry point
        assert _max_rel(y, y_or) <= TOL             # the oracle
    # same kernel, same inputs, fixed reduction order: the two calls agree bit for bit
    assert torch.equal(outs[0], outs[1])


def test_noalloc_batch_that_fits_runs_on_the_batched_kernel():
    """M = 16 at 1024 x 4096: the batched kernel's re-tiled activations and partial sums fit the 4 MiB array."""
    import sbvr  # noqa: F401
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    N, K, S, C, M = 1024, 4096, 4, 4096, 16
    w = _packed(N, K, S, C, 21, dev)
    x = torch.randn((M, K), device=dev).half()
    y_ref = torch.empty((M, N), dtype=torch.float16, device=dev)
    assert _call_regular(_lib, x, w, y_ref, M, N, K, S, C) == 0
    for _ in range(2):
        y = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
        rc = _call_noalloc(L, x, w, y, M, N, K, S, C)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        assert _max_rel(y, y_ref) <= TOL
        assert _max_rel(y, _oracle(x, w)) <= TOL


def test_noalloc_refuses_what_cannot_fit():
    """M = 2048 at 4096 x 14336 needs 56 MiB of re-tiled activations: refused with SBVR_ERR_NOALLOC_LIMIT, nothing launched."""
    import sbvr  # noqa: F401
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    N, K, S, C, M = 4096, 14336, 4, 256, 2048
    w = _packed(N, K, S, C, 13, dev)
    x = torch.randn((M, K), device=dev).half()
    y = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
    rc = _call_noalloc(L, x, w, y, M, N, K, S, C)
    assert rc == -8, _lib.strerror(rc)
    assert "4 MiB" in _lib.strerror(rc)
    torch.cuda.synchronize()
    assert torch.isnan(y).all()                     # the output was not touched


def test_noalloc_argument_errors():
    import sbvr  # noqa: F401
    from sbvr import _lib
    L = _lib.lib
    buf = torch.zeros(1024, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    assert L.sbvr_linear_f16_noalloc(None, p, p, 1, p, 4, None, p, 1, 64, 256, 4, 256, None) == -1
    assert L.sbvr_linear_f16_noalloc(p, p, p, 1, p, 4, None, p, 1, 64, 300, 4, 256, None) == -2
    assert L.sbvr_linear_f16_noalloc(p, p, p, 1, p, 4, None, p, 1, 64, 256, 9, 256, None) == -1
