"""The pushed all-reduce of the tensor-parallel decode step on ONE GPU: two "ranks" are two calls of
`sbvr_linear_push_f16` (each with its own column shard of the weight) whose peer list points twice at the same local
receive area, followed by `sbvr_ll_reduce_add_rmsnorm_f16` with world = 2.  Nothing waits on anything that does not
come: the calls run one after the other on one stream.  A second test leaves rank 1 out and checks that the bounded wait
of the receiving kernel runs out, is reported through the workspace status and leaves the workspace usable.
"""
import ctypes
import time

import numpy as np
import pytest
import torch

from oracle import sbvr_oracle as O

pytestmark = pytest.mark.gpu


def _shard(N, K, S, seed, dev):
    import sbvr
    p = O.make_packed(N, K, S, G=256, mode="u16", C=4096, seed=seed)
    idx = torch.from_numpy(p["coeff_idx"].view(np.int16)).view(torch.uint16)
    w = sbvr.sbvr.from_packed(torch.from_numpy(p["bvr"].view(np.int32)), idx, torch.from_numpy(p["coeff"]), group_len=256,
                              device=dev)
    return p, w


def _desc(recv, step, cps, call, rank, world, rows_max, dev):
    """An sbvr_push_desc_t in device memory whose peers are all the one local receive area."""
    from sbvr import _lib
    d = _lib.PushDesc()
    for r in range(world):
        d.peer_recv[r] = recv.data_ptr()
    d.step = step.data_ptr()
    d.calls_per_step, d.call_idx, d.rank, d.world, d.rows_max = cps, call, rank, world, rows_max
    return torch.frombuffer(bytearray(bytes(d)), dtype=torch.uint8).to(dev)


def _push(L, ws, st, x_op, x, w, desc, M, N, K):
    b, ix, ib, c, C = w._abi_args()
    return L.sbvr_linear_push_f16(x_op, x.data_ptr(), None, None, None, ctypes.c_float(0.0), b, ix, ib, c, C, None,
                                  desc.data_ptr(), M, N, K, w.num_sums, w.bvr_len, ws.handle, st)


@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("silu", [False, True])
def test_pushed_partials_are_reduced_like_separate_kernels(M, silu):
    import sbvr
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    N, Kr, world, rows_max, cps = 1024, 1536, 2, 4, 4
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(torch.cuda.current_device(), st)
    recv = torch.zeros(2 * world * rows_max * (N // 2), dtype=torch.int64, device=dev)
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    rng = np.random.default_rng(M)
    shards = [_shard(N, Kr, 4, 40 + r, dev) for r in range(world)]
    h = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float16)).to(dev)
    weight = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(N)).astype(np.float16)).to(dev)
    for it in range(6):                                   # consecutive calls alternate the two slots; epochs grow
        call = it % cps
        xs, parts = [], []
        for r in range(world):
            if silu:
                gu = torch.from_numpy(rng.standard_normal((M, 2 * Kr)).astype(np.float16)).to(dev)
                act = torch.empty((M, Kr), dtype=torch.float16, device=dev)
                assert L.sbvr_silu_mul_f16(gu.data_ptr(), act.data_ptr(), M, Kr, st) == 0
                xs.append(gu)
                parts.append(sbvr.linear(act, shards[r][1]))
            else:
                x = torch.from_numpy(rng.standard_normal((M, Kr)).astype(np.float16)).to(dev)
                xs.append(x)
                parts.append(sbvr.linear(x, shards[r][1]))
        for r in range(world):
            desc = _desc(recv, step, cps, call, r, world, rows_max, dev)
            rc = _push(L, ws, st, 1 if silu else 0, xs[r], shards[r][1], desc, M, N, Kr)
            assert rc == 0, _lib.strerror(rc)
        h_out = torch.empty_like(h)
        y = torch.empty_like(h)
        rc = L.sbvr_ll_reduce_add_rmsnorm_f16(recv.data_ptr(), step.data_ptr(), cps, call, world, rows_max, h.data_ptr(),
                                              weight.data_ptr(), h_out.data_ptr(), y.data_ptr(), M, N, ctypes.c_float(1e-5),
                                              1 if it % 2 == 0 else 0, ws.handle, st)
        assert rc == 0, _lib.strerror(rc)
        assert ws.status(st) == 0
        # the same arithmetic with the separate kernels' results: fp32 sum of the fp16 partials in rank order, one rounding
        delta = (parts[0].float() + parts[1].float()).half()
        h_ref = h + delta
        y_ref = torch.empty_like(h)
        assert L.sbvr_add_rmsnorm_f16(h.data_ptr(), delta.data_ptr(), weight.data_ptr(), None, y_ref.data_ptr(), M, N,
                                      ctypes.c_float(1e-5), st) == 0
        torch.cuda.synchronize()
        assert torch.equal(h_out, h_ref)
        # the mean square is summed in another order than in the separate kernel: a last-bit difference is possible
        assert torch.allclose(y.float(), y_ref.float(), rtol=2e-3, atol=1e-3)
        h = h_out
        if call == cps - 1:
            step += 1


def test_missing_rank_runs_into_the_bounded_wait():
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    N, Kr, world, rows_max, cps, M = 1024, 1024, 2, 4, 2, 1
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(torch.cuda.current_device(), st)
    assert ws.status(st) == 0
    recv = torch.zeros(2 * world * rows_max * (N // 2), dtype=torch.int64, device=dev)
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    p, w = _shard(N, Kr, 4, 9, dev)
    x = torch.randn((M, Kr), device=dev).half()
    desc = _desc(recv, step, cps, 0, 0, world, rows_max, dev)
    assert _push(L, ws, st, 0, x, w, desc, M, N, Kr) == 0      # rank 1 never pushes
    h = torch.randn((M, N), device=dev).half()
    weight = torch.ones(N, dtype=torch.float16, device=dev)
    h_out, y = torch.empty_like(h), torch.empty_like(h)
    t0 = time.perf_counter()
    rc = L.sbvr_ll_reduce_add_rmsnorm_f16(recv.data_ptr(), step.data_ptr(), cps, 0, world, rows_max, h.data_ptr(),
                                          weight.data_ptr(), h_out.data_ptr(), y.data_ptr(), M, N, ctypes.c_float(1e-5),
                                          1, ws.handle, st)
    assert rc == 0
    status = ws.status(st)
    assert status == -6, _lib.strerror(status)            # SBVR_ERR_TIMEOUT
    assert time.perf_counter() - t0 < 10.0
    assert ws.status(st) == 0
    # the workspace serves an ordinary call afterwards
    import sbvr
    yy = sbvr.linear(x, w).cpu().numpy()
    ref = O.linear_c(x.cpu().numpy(), p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    assert O.max_rel_err(yy, ref) <= 1e-2


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("pushed", [True, False])
def test_reduce_kernels_leave_the_digits_of_the_next_gemv(M, pushed):
    """emit_digits: the all-reduce + RMSNorm kernel also writes its result as the activation digits of the decode GEMV into
    the workspace, and the following sbvr_linear_fused_f16(SBVR_XOP_DIGITS) gives the bits of the ordinary linear on y."""
    import sbvr
    from sbvr import _lib
    from sbvr.core import XOP_DIGITS, linear_fused
    L = _lib.lib
    dev = torch.device("cuda")
    H, Kr, N2, world, rows_max, cps = 2048, 1024, 768, 2, 4, 2
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(torch.cuda.current_device(), st)
    rng = np.random.default_rng(10 + M)
    shards = [_shard(H, Kr, 4, 60 + r, dev) for r in range(world)]
    _, w2 = _shard(N2, H, 4, 70, dev)
    h = torch.from_numpy(rng.standard_normal((M, H)).astype(np.float16)).to(dev)
    weight = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(H)).astype(np.float16)).to(dev)
    xs = [torch.from_numpy(rng.standard_normal((M, Kr)).astype(np.float16)).to(dev) for _ in range(world)]
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    h_out, y = torch.empty_like(h), torch.empty_like(h)
    if pushed:
        recv = torch.zeros(2 * world * rows_max * (H // 2), dtype=torch.int64, device=dev)
        for r in range(world):
            assert _push(L, ws, st, 0, xs[r], shards[r][1], _desc(recv, step, cps, 0, r, world, rows_max, dev), M, H, Kr) == 0
        rc = L.sbvr_ll_reduce_add_rmsnorm_digits_f16(recv.data_ptr(), step.data_ptr(), cps, 0, world, rows_max, h.data_ptr(),
                                                     weight.data_ptr(), h_out.data_ptr(), y.data_ptr(), M, H,
                                                     ctypes.c_float(1e-5), 1, 1, ws.handle, st)
    else:
        # one-shot form with a world of one: this rank's partial is the sum of the two shards' results
        part = (sbvr.linear(xs[0], shards[0][1]).float() + sbvr.linear(xs[1], shards[1][1]).float()).half()
        buf = torch.zeros(2 * M * H, dtype=torch.float16, device=dev)
        buf[:M * H] = part.reshape(-1)
        flags = torch.zeros(4, dtype=torch.int32, device=dev)
        bufs = torch.tensor([buf.data_ptr()], dtype=torch.int64, device=dev)
        fl = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=dev)
        rc = L.sbvr_allreduce_add_rmsnorm_digits_f16(bufs.data_ptr(), fl.data_ptr(), step.data_ptr(), cps, 0, 0, 1,
                                                     ctypes.c_size_t(M * H), h.data_ptr(), weight.data_ptr(), h_out.data_ptr(),
                                                     y.data_ptr(), M, H, ctypes.c_float(1e-5), 1, ws.handle, st)
    assert rc == 0, _lib.strerror(rc)
    out = torch.empty((M, N2), dtype=torch.float16, device=dev)
    assert linear_fused(XOP_DIGITS, y, w2, out)
    torch.cuda.synchronize()
    assert ws.status(st) == 0
    ref = sbvr.linear(y, w2)
    assert torch.equal(out, ref)
