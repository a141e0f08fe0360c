"""A bounded device-side wait that runs out, made on the host: nothing faults, traps or hangs.

`sbvr_allreduce_add_rmsnorm_f16` is called on ONE GPU as rank 0 of a world of two whose "peer" buffer and flag
arrays are ordinary local allocations, and nobody ever raises rank 1's flag.  The kernel polls for it a bounded number
of times (about a third of a second), records the time-out in the workspace status words and returns; the host then
reads SBVR_ERR_TIMEOUT from `sbvr_workspace_status`, which also clears the workspace, and the next ordinary call on the
same workspace gives a correct result.
"""
import ctypes
import time

import numpy as np
import pytest
import torch

from oracle import sbvr_oracle as O

pytestmark = pytest.mark.gpu


def test_allreduce_wait_runs_out_and_the_workspace_recovers():
    import sbvr
    from sbvr import _lib
    L = _lib.lib
    dev = torch.device("cuda")
    rows, hidden, world = 1, 1024, 2
    buf_elems = rows * hidden
    bufs = [torch.zeros(2 * buf_elems, dtype=torch.float16, device=dev) for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    peer_bufs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    h_in = torch.randn((rows, hidden), device=dev).half()
    weight = torch.ones(hidden, dtype=torch.float16, device=dev)
    h_out = torch.empty_like(h_in)
    y = torch.empty_like(h_in)
    st = torch.cuda.current_stream().cuda_stream
    ws = _lib.workspace(torch.cuda.current_device(), st)
    assert ws.status(st) == 0                                   # clean to begin with
    t0 = time.perf_counter()
    rc = L.sbvr_allreduce_add_rmsnorm_f16(peer_bufs.data_ptr(), peer_flags.data_ptr(), step.data_ptr(), 2, 0, 0, world,
                                          ctypes.c_size_t(buf_elems), h_in.data_ptr(), weight.data_ptr(), h_out.data_ptr(),
                                          y.data_ptr(), rows, hidden, ctypes.c_float(1e-5), ws.handle, st)
    assert rc == 0, _lib.strerror(rc)                           # the launch itself succeeds
    status = ws.status(st)                                      # synchronises the stream, reads and clears the status
    waited = time.perf_counter() - t0
    assert status == -6, _lib.strerror(status)                  # SBVR_ERR_TIMEOUT
    assert waited < 10.0, waited                                # bounded: well under the 2^22 polls' worst case
    assert int(flags[0][0].item()) == 1                         # rank 0 did publish its own epoch to itself ...
    assert int(flags[1][0].item()) == 1                         # ... and to its "peer"; the peer never answered
    assert ws.status(st) == 0                                   # reading the status cleared it

    # the same workspace serves an ordinary call afterwards
    N, K, S = 256, 1024, 4
    p = O.make_packed(N, K, S, G=256, mode="u8", seed=5)
    w = sbvr.sbvr.from_packed(torch.from_numpy(p["bvr"].view(np.int32)), torch.from_numpy(p["coeff_idx"]),
                              torch.from_numpy(p["coeff"]), group_len=256, device=dev)
    x = np.random.default_rng(3).standard_normal((1, K)).astype(np.float16)
    yy = sbvr.linear(torch.from_numpy(x).to(dev), w).cpu().numpy()
    ref = O.linear_c(x, p["bvr"], p["coeff_idx"], p["coeff"], G=256)
    assert O.max_rel_err(yy, ref) <= 1e-2
    assert ws.status(st) == 0
