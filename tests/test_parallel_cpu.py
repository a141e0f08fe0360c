"""Tensor-parallel slicing of packed weights, on CPU: two gloo ranks hold one shard each, compute their part with
the oracle and exchange exactly what the GPU model exchanges (all-gather for column-parallel linears, all-reduce
for row-parallel ones).  No GPU, no CUDA library."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _packed(N, K, S, G, C, seed):
    from oracle import sbvr_oracle as O
    p = O.make_packed(N, K, S, G=G, mode="u8" if C <= 256 else "u16", C=C, seed=seed)
    idx = p["coeff_idx"]
    idx_t = torch.from_numpy(idx) if idx.dtype == np.uint8 else torch.from_numpy(idx.view(np.int16)).view(torch.uint16)
    return p, {"bvr": torch.from_numpy(p["bvr"].view(np.int32)), "coeff_idx": idx_t, "coeff_cache": torch.from_numpy(p["coeff"])}


def _np(t):
    bvr = t["bvr"].numpy().view(np.uint32)
    idx = t["coeff_idx"]
    idx = idx.numpy() if idx.dtype == torch.uint8 else idx.view(torch.int16).numpy().view(np.uint16)
    return bvr, idx, t["coeff_cache"].numpy()


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "sbvr-cpu-arm_b200"))
    from models import parallel
    from oracle import sbvr_oracle as O
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, K, S, G = 256, 1024, 4, 256
        p, t = _packed(N, K, S, G, 256, 11)
        x = np.random.default_rng(3).standard_normal((2, K)).astype(np.float16)
        full = O.linear(x, p["bvr"], p["coeff_idx"], p["coeff"], G=G).astype(np.float32)
        # column-parallel: every rank computes its rows; all-gather restores the full output
        b, i, c = _np(parallel.shard_rows(t, rank, world))
        part = torch.from_numpy(O.linear(x, b, i, c, G=G).astype(np.float32))
        got = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(got, part)
        col = torch.cat(got, dim=1).numpy()
        # row-parallel: every rank multiplies its slice of the input; all-reduce sums the partial products
        b, i, c = _np(parallel.shard_cols(t, rank, world, G))
        k0, k1 = rank * K // world, (rank + 1) * K // world
        partial = torch.from_numpy(O.linear_f64(x[:, k0:k1], b, i, c, G=G).astype(np.float64))
        dist.all_reduce(partial)
        ref64 = O.linear_f64(x, p["bvr"], p["coeff_idx"], p["coeff"], G=G)
        ok_col = bool(np.array_equal(col, full))
        ok_row = bool(np.abs(partial.numpy() - ref64).max() <= 1e-9 * np.abs(ref64).max())
        if rank == 0:
            out.put((ok_col, ok_row))
    finally:
        dist.destroy_process_group()


def test_two_rank_shards_recombine():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = q.get(timeout=180)
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    assert res == (True, True)


def test_fuse_rows_offsets_codebooks():
    sys.path.insert(0, os.path.join(ROOT, "sbvr-cpu-arm_b200"))
    from models import parallel
    from oracle import sbvr_oracle as O
    pa, ta = _packed(64, 512, 4, 256, 256, 1)
    pb, tb = _packed(32, 512, 4, 256, 256, 2)
    fused = parallel.fuse_rows([ta, tb, ta])
    assert fused["coeff_cache"].shape[0] == 512            # ta's codebook is kept once
    assert fused["coeff_idx"].dtype == torch.uint16
    b, i, c = _np(fused)
    W = O.decode(b, i, c, G=256)
    Wa = O.decode(pa["bvr"], pa["coeff_idx"], pa["coeff"], G=256)
    Wb = O.decode(pb["bvr"], pb["coeff_idx"], pb["coeff"], G=256)
    assert np.array_equal(W.view(np.uint16), np.concatenate([Wa, Wb, Wa]).view(np.uint16))


def test_presets_split_over_the_rank_counts_they_are_used_with():
    """The model presets the multi-GPU tests and bench.py run at 2, 4 and 8 ranks split over them: heads, KV heads,
    vocabulary rows, and whole 256-column groups in the inputs of the row-parallel projections."""
    sys.path.insert(0, os.path.join(ROOT, "sbvr-cpu-arm_b200"))
    from models.sbvr_llama import LlamaConfig
    for preset, worlds in (("tiny", (1, 2)), ("tiny8", (1, 2, 4, 8)), ("8b", (1, 2, 4, 8)), ("70b", (1, 2, 4, 8))):
        cfg = LlamaConfig.preset(preset)
        for world in worlds:
            assert cfg.tp_problems(world) == [], (preset, world, cfg.tp_problems(world))
    assert LlamaConfig.preset("tiny").tp_problems(8)          # 512 hidden columns are not eight groups of 256
