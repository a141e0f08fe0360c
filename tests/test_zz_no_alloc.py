"""The allocation-free entry point `sbvr_linear_f16_noalloc`, called through the C ABI.

It exists for callers that are forbidden to allocate device memory (a serving process that owns the whole GPU
arena, a latency-critical loop, code next to an open stream capture): it takes no workspace and keeps its scratch
in a fixed array inside the library.  The test checks that it gives the same result as the regular entry point
`sbvr_linear_f16`, on two calls in a row (the second call meets whatever the first left in the shared array), that
it copes with a different problem in between, and that it refuses a problem whose scratch cannot fit.

The file name sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2          # same tolerance as tests/test_gpu_parity.py: max|a - b| / max|b|


def _packed(N, K, S, C, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    bvr = torch.randint(-2**31, 2**31 - 1, (K // 32, N, S), dtype=torch.int32, device=dev, generator=g)
    idx = torch.randint(0, C, (K // 256, N), device=dev, generator=g)
    idx = idx.to(torch.uint8) if C <= 256 else idx.to(torch.int16)
    cache = (torch.randn((C, S), device=dev, generator=g) * 0.01).half()
    return bvr, idx, cache


def _max_rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def _call_noalloc(L, x, w, y, M, N, K, S, C, bias=None):
    bvr, idx, cache = w
    st = torch.cuda.current_stream().cuda_stream
    return L.sbvr_linear_f16_noalloc(x.data_ptr(), bvr.data_ptr(), idx.data_ptr(), idx.element_size(), cache.data_ptr(),
                                     C, None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K, S, 256, st)


def _call_regular(_lib, x, w, y, M, N, K, S, C, bias=None):
    bvr, idx, cache = w
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(torch.cuda.current_device(), st)
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

    before = torch.cuda.memory_allocated()
    outs = []
    for call in range(2):
        y = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
        rc = _call_noalloc(L, x, w, y, M, N, K, S, C, bias)
        assert rc == 0, _lib.strerror(rc)
        outs.append(y)
        if call == 0:
            y2 = torch.full((2, N2), float("nan"), dtype=torch.float16, device=dev)
            rc = _call_noalloc(L, x2, w2, y2, 2, N2, K2, 3, 200)
            assert rc == 0, _lib.strerror(rc)
            torch.cuda.synchronize()
            assert _max_rel(y2, y2_ref) <= TOL
    torch.cuda.synchronize()
    for y in outs:
        assert torch.isfinite(y).all()
        assert _max_rel(y, y_ref) <= TOL
    # same kernel, same inputs, fixed reduction order: the two calls agree bit for bit
    assert torch.equal(outs[0], outs[1])
    assert torch.cuda.memory_allocated() - before <= 3 * M * N * 2 + 2 * N2 * 2 + 4096   # only the test's own outputs


def test_noalloc_refuses_what_cannot_fit():
    """262 144 output rows at M = 4 need more than 4 MiB of partial sums: refused before any launch.  Should a later
    kernel need less scratch and accept it, the result must simply be right."""
    import sbvr  # noqa: F401
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    N, K, S, C, M = 262144, 256, 4, 256, 4
    w = _packed(N, K, S, C, 13, dev)
    x = torch.randn((M, K), device=dev).half()
    y = torch.zeros((M, N), dtype=torch.float16, device=dev)
    rc = _call_noalloc(L, x, w, y, M, N, K, S, C)
    assert rc in (0, -8), _lib.strerror(rc)
    if rc == -8:
        assert "4 MiB" in _lib.strerror(rc)
    else:
        y_ref = torch.empty_like(y)
        assert _call_regular(_lib, x, w, y_ref, M, N, K, S, C) == 0
        torch.cuda.synchronize()
        assert _max_rel(y, y_ref) <= TOL


def test_noalloc_argument_errors():
    import sbvr  # noqa: F401
    from sbvr import _lib
    L = _lib.lib
    buf = torch.zeros(1024, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    assert L.sbvr_linear_f16_noalloc(None, p, p, 1, p, 4, None, p, 1, 64, 256, 4, 256, None) == -1
    assert L.sbvr_linear_f16_noalloc(p, p, p, 1, p, 4, None, p, 1, 64, 300, 4, 256, None) == -2
    assert L.sbvr_linear_f16_noalloc(p, p, p, 1, p, 4, None, p, 1, 64, 256, 9, 256, None) == -1
