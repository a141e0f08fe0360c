#!/usr/bin/env python
"""Benchmark of the SBVR decode-time linear (GEMV, M = 1) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (the GEMV / small-M sweep configuration at its headline point): one STEP = the seven SBVR linears of a
Llama-3-8B decoder layer at batch 1 -- q, o (4096x4096), k, v (1024x4096), gate, up (14336x4096),
down (4096x14336) -- 4 bit-planes, group 256, uint16 codebook of 4096 lines, fp16 activations.
Weights are seeded synthetic packed tensors in the reference layout (Bernoulli(0.5) planes,
N(0, 0.01) codebook); activations N(0, 1).  Four distinct layers (444 MB of packed weights) are
cycled, so every step streams weights that left L2 (126 MB) long ago.

metric `sbvr_gemv_hbm_gbs_m1` = algorithmic bytes of a step (planes + indices + codebook + x + y,
111.1 MB) / time of a step, summed over GPUs.  With N > 1 every rank runs the same per-GPU work on
its own weights (output-row shards of an N-times larger layer stack): no data-path collective,
weak scaling; time = max over ranks.  The timed region (--steps steps) is repeated 11 times and the
median is reported.  At N > 1 the line also carries `strong_rows` (ONE layer's rows split over the
ranks) and `tp_parity` (tensor-parallel logits against one rank), and the Llama decode sections run
tensor parallel over all ranks.

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "sbvr-cpu-arm_b200"))

SHAPES = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
          ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
S, G, C, IDXB = 4, 256, 4096, 2
N_LAYERS = 4
REPEATS = 11                  # repeats of every timed region; the median is reported, min and max beside it
# dram__bytes_read.sum + dram__bytes_write.sum of one linear_tcs_kernel launch at 14336x4096 (ncu, see profiles/)
TRAFFIC_DOMINANT = 29_920_000


def alg_bytes(M, N, K, s=S, g=G, ib=IDXB, c=C):
    """Algorithmic bytes of one linear: planes + group indices + codebook + activations + result."""
    return N * K * s // 8 + N * (K // g) * ib + c * s * 2 + M * K * 2 + M * N * 2


STEP_BYTES = sum(alg_bytes(1, n, k) for _, n, k in SHAPES)


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_layer(torch, dev, gen):
    import sbvr
    layer = {}
    for name, N, K in SHAPES:
        bvr = torch.randint(-2**31, 2**31 - 1, (K // 32, N, S), dtype=torch.int32, device=dev, generator=gen)
        idx = torch.randint(0, C, (K // G, N), device=dev, generator=gen).to(torch.int16).view(torch.uint16)
        cache = torch.randn((C, S), device=dev, generator=gen) * 0.01
        order = cache.abs().argsort(dim=1)
        cache = torch.gather(cache, 1, order).half()
        layer[name] = sbvr.sbvr.from_packed(bvr, idx, cache, group_len=G, device=dev)
    return layer


def run_ours(args):
    import torch
    import sbvr
    from sbvr import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    layers = [make_layer(torch, dev, gen) for _ in range(N_LAYERS)]
    x_h = torch.randn((1, 4096), device=dev, generator=gen).half()
    x_i = torch.randn((1, 14336), device=dev, generator=gen).half()
    outs = {name: torch.empty((1, n), dtype=torch.float16, device=dev) for name, n, _ in SHAPES}

    def step(li):
        L = layers[li % N_LAYERS]
        for name, _, k in SHAPES:
            sbvr.linear(x_h if k == 4096 else x_i, L[name], None, out=outs[name])

    stream = torch.cuda.Stream(device=dev)
    graphs = []
    with torch.cuda.stream(stream):
        for li in range(N_LAYERS):
            step(li)                                   # creates the workspace, sets kernel attributes
        torch.cuda.synchronize()
        for li in range(N_LAYERS):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step(li)
            graphs.append(g)
        for i in range(max(args.warmup, 3)):
            graphs[i % N_LAYERS].replay()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        # the timed region (exactly --steps steps between two events) is repeated; the median repeat is reported
        rep_ms = []
        for rep in range(REPEATS):
            if dist:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(args.steps):
                graphs[i % N_LAYERS].replay()
            e1.record(stream)
            e1.synchronize()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if dist:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            rep_ms.append(ms)
        if dist:
            dist.barrier()
        clocks = sampler.stop() if rank == 0 else None
        ms = sorted(rep_ms)[len(rep_ms) // 2]

        # ---- the dominant kernel alone (gate/up shape): one launch per linear
        Nd, Kd = 14336, 4096
        copies = [layers[i][n] for i in range(N_LAYERS) for n in ("gate", "up")]      # 8 x 29.4 MB > L2
        st = stream.cuda_stream
        ws = _lib.workspace(local, st)
        yd = outs["gate"]

        def dom(i):
            b, ix, ib, c, cc = copies[i % len(copies)]._abi_args()
            _lib.check(_lib.lib.sbvr_linear_f16(x_h.data_ptr(), b, ix, ib, c, cc, None, yd.data_ptr(), 1, Nd, Kd, S, G,
                                                2, ws.handle, st))
        for i in range(len(copies)):
            dom(i)
        reps = 5 * len(copies)
        gd = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gd, stream=stream):
            for i in range(reps):
                dom(i)
        gd.replay()
        torch.cuda.synchronize()
        dom_all = []
        for _ in range(REPEATS):
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            d0.record(stream)
            gd.replay()
            d1.record(stream)
            d1.synchronize()
            dom_all.append(d0.elapsed_time(d1) * 1e3 / reps)
        dom_us = sorted(dom_all)[len(dom_all) // 2]

        # ---- end to end through the public API with host buffers (copies inside the timed region)
        # the step's activations (hidden-sized and intermediate-sized row) sit in one pinned host buffer, its seven results
        # land in one pinned host buffer: one copy each way per step, the linears write into views of the device buffer
        n_in = x_h.numel() + x_i.numel()
        n_out = sum(n for _, n, _ in SHAPES)
        x_host = torch.cat((x_h.view(-1), x_i.view(-1))).cpu().pin_memory()
        y_host = torch.empty(n_out, dtype=torch.float16).pin_memory()
        x_dev = torch.empty(n_in, dtype=torch.float16, device=dev)
        y_dev = torch.empty(n_out, dtype=torch.float16, device=dev)
        xh_dev, xi_dev = x_dev[:x_h.numel()].view(1, -1), x_dev[x_h.numel():].view(1, -1)
        y_view, off = {}, 0
        for name, n, _ in SHAPES:
            y_view[name] = y_dev[off:off + n].view(1, n)
            off += n

        def e2e_body(li):
            x_dev.copy_(x_host, non_blocking=True)
            L = layers[li % N_LAYERS]
            for name, _, k in SHAPES:
                sbvr.linear(xh_dev if k == 4096 else xi_dev, L[name], None, out=y_view[name])
            y_host.copy_(y_dev, non_blocking=True)
        # one CUDA graph per layer holds the step as a user would issue it: pinned host -> device copy of the
        # activations, the seven linears, device -> pinned host copy of the results; a step = replay + wait
        e2e_graphs = []
        for li in range(N_LAYERS):
            e2e_body(li)
            stream.synchronize()
            ge = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ge, stream=stream):
                e2e_body(li)
            e2e_graphs.append(ge)

        def e2e_step(li):
            e2e_graphs[li % N_LAYERS].replay()
            stream.synchronize()
        for i in range(3):
            e2e_step(i)
        if dist:
            dist.barrier()
        n_e2e = min(args.steps, 64)
        t0 = time.perf_counter()
        for i in range(n_e2e):
            e2e_step(i)
        e2e_s = time.perf_counter() - t0
        if dist:
            t = torch.tensor([e2e_s], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
    extra = {}
    if world > 1:
        extra["strong_rows"] = strong_rows(torch, dev, dist, world, stream, gen)
        extra["tp_parity"] = tp_parity(torch, dev, dist, world)
    if not args.no_extras:
        if world == 1:
            extra.update(small_m_and_prefill(torch, dev, stream))
        def decode_section(*a):
            # one rank: a failing section is reported, the line is still printed (with several ranks an exception on one
            # of them must end the job: the others wait in collectives)
            if dist:
                return llama_decode(torch, dev, dist, world, *a)
            try:
                return llama_decode(torch, dev, dist, world, *a)
            except Exception as e:
                torch.cuda.empty_cache()
                return {"model": a[0], "batch": a[1], "error": str(e)[:200]}
        decodes = [decode_section("8b", 1, 512, 256)]
        if not args.skip_70b:
            decodes.append(decode_section("70b", 1, 1024, 256))
            decodes.append(decode_section("70b", 16, 1024, 64))
        extra["llama_decode"] = decodes
    for (d, s_), w in _lib._workspaces.items():
        assert w.status(s_) == 0, "a device-side wait timed out during the benchmark"

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak()
    ms_per_step = ms / args.steps
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9
    dom_bytes = alg_bytes(1, Nd, Kd)
    achieved = dom_bytes / (dom_us * 1e-6) / 1e9
    h2d = (4096 + 14336) * 2
    d2h = sum(n for _, n, _ in SHAPES) * 2
    line = {
        "metric": "sbvr_gemv_hbm_gbs_m1", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5),
        "repeats": {"n": REPEATS, "statistic": "median", "ms_per_step_min": round(min(rep_ms) / args.steps, 5),
                    "ms_per_step_max": round(max(rep_ms) / args.steps, 5)},
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama3-8b decoder-layer linears (q,k,v,o,gate,up,down), M=1, S=4, G=256, "
                               "u16 codebook C=4096", "bytes_per_step": STEP_BYTES,
                   "l2": "inputs larger than L2: 4 layers = 444 MB of packed weights cycled",
                   "launch": "CUDA graph per layer: 7 linears = 8 kernels (the K = 14336 linear quantises its activations in a "
                             "small kernel of its own, the K = 4096 ones inside the GEMV)", "parallelism": f"rows x{world}"},
        "roofline": {"bound": "hbm", "kernel": "linear_tcs_kernel<S=4,G=256,M=1,u16,KS=2> 14336x4096",
                     "achieved": round(achieved, 1), "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "us_per_launch": round(dom_us, 2), "us_per_launch_min": round(min(dom_all), 2),
                     "us_per_launch_max": round(max(dom_all), 2), "bytes_per_launch": dom_bytes, "traffic": TRAFFIC_DOMINANT},
        "e2e": {"value": round(world * STEP_BYTES / (e2e_s / n_e2e) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s / n_e2e * 1e3, 4),
                "api": "sbvr.linear (python) -> sbvr_linear_f16 (C ABI), pinned host x in, pinned host y out; the step "
                       "(1 H2D copy of both activation rows, 7 linears, 1 D2H copy of the 7 results) is captured once and "
                       "replayed, then the stream is waited for"},
        "gpu_launches": args.steps * (len(SHAPES) + 1),
        "gpu_launches_note": f"per timed region of {args.steps} steps (8 kernels per step); the region is repeated {REPEATS} times",
        "clocks": clocks,
    }
    line.update(extra)
    line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def strong_rows(torch, dev, dist, world, stream, gen):
    """Strong scaling of ONE layer: every linear's output rows are split over the ranks (what the column-parallel
    projections of a tensor-parallel model launch), no collective.  Aggregate GB/s = bytes of the whole layer / time of the
    slowest rank; enough shard layers are cycled to exceed L2."""
    import sbvr
    shard = [(name, n // world, k) for name, n, k in SHAPES]
    layer_bytes = sum(alg_bytes(1, n, k) for _, n, k in shard)
    n_layers = max(4, int(2 * 126e6 / layer_bytes) + 1)

    def mk(N, K):
        bvr = torch.randint(-2**31, 2**31 - 1, (K // 32, N, S), dtype=torch.int32, device=dev, generator=gen)
        idx = torch.randint(0, C, (K // G, N), device=dev, generator=gen).to(torch.int16).view(torch.uint16)
        cache = (torch.randn((C, S), device=dev, generator=gen) * 0.01).half()
        return sbvr.sbvr.from_packed(bvr, idx, cache, group_len=G, device=dev)
    layers = [{name: mk(n, k) for name, n, k in shard} for _ in range(n_layers)]
    xs = {k: torch.randn((1, k), device=dev, generator=gen).half() for k in {k for _, _, k in shard}}
    outs = {name: torch.empty((1, n), dtype=torch.float16, device=dev) for name, n, _ in shard}
    with torch.cuda.stream(stream):
        def step(L):
            for name, _, k in shard:
                sbvr.linear(xs[k], L[name], None, out=outs[name])
        for L in layers:
            step(L)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for L in layers:
                step(L)
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(REPEATS):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            e1.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append(float(t.item()) * 1e3 / n_layers)
    us = sorted(times)[len(times) // 2]
    del layers
    torch.cuda.empty_cache()
    return {"what": "one llama3-8b layer, every linear's rows split over the ranks, M=1, no collective",
            "us_per_layer": round(us, 2), "GBps_aggregate": round(STEP_BYTES / us / 1e3, 1),
            "shard_shapes": [[n, k] for _, n, k in shard], "layers_cycled": n_layers}


def tp_parity(torch, dev, dist, world):
    """Correctness of the tensor-parallel model on this job's ranks: logits of a small model against the same model on one
    rank (max relative error, rank 0), graph = eager tokens, and token agreement of the fused all-reduce path with NCCL."""
    from models.sbvr_llama import LlamaConfig, SBVRLlamaForCausalLM
    cfg = LlamaConfig.preset("tiny8")                   # three sequences: the decode rows also take the digit hand-over
    if cfg.tp_problems(world):                          # the same on every rank: nobody is left waiting in a collective
        return {"skipped": "; ".join(cfg.tp_problems(world))}
    tp = SBVRLlamaForCausalLM(cfg, device=dev, tp_group=dist.group.WORLD, max_batch=3, max_ctx=64).init_synthetic(3)
    ids = torch.randint(0, cfg.vocab_size, (3, 24), device=dev, generator=torch.Generator(device=dev).manual_seed(9))
    logits = tp(ids).float()
    a = tp.generate(ids, 10, use_graph=False)
    b = tp.generate(ids, 10, use_graph=True)
    res = {"model": "tiny8", "tp": world, "graph_equals_eager": bool(torch.equal(a, b))}
    if tp.enable_fused_allreduce(16):
        c = tp.generate(ids, 10, use_graph=True)
        res["fused_vs_nccl_token_agreement"] = round((c == a).float().mean().item(), 4)
    else:
        res["fused_allreduce"] = "unavailable: " + str(getattr(tp, "_comm_error", "?"))[:100]
    err = torch.zeros(1, device=dev)
    if dist.get_rank() == 0:
        one = SBVRLlamaForCausalLM(cfg, device=dev, max_batch=3, max_ctx=64).init_synthetic(3)
        ref = one(ids).float()
        err[0] = (logits - ref).abs().max() / ref.abs().max()
        del one
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    res["logits_max_rel_err_vs_one_rank"] = round(float(err.item()), 5)
    res["tolerance"] = 1e-2
    tp._check()
    del tp
    torch.cuda.empty_cache()
    return res


def graph_time_us(torch, stream, fns, reps=5):
    """Average device time of one call of the functions in `fns`, replayed from one CUDA graph."""
    with torch.cuda.stream(stream):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        e1.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps / len(fns)


def median_graph_time_us(torch, stream, fns, reps=5, repeats=5):
    """Median over `repeats` of graph_time_us-style measurements (one graph, `reps` replays per measurement)."""
    with torch.cuda.stream(stream):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        out = []
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            e1.synchronize()
            out.append(e0.elapsed_time(e1) * 1e3 / reps / len(fns))
    return sorted(out)[len(out) // 2]


def small_m_and_prefill(torch, dev, stream):
    """The neighbouring configurations beside the headline: the M sweep of the layer shapes for 2, 3 and 4 bit-planes
    (HBM roofline), the same at group length 128 with direct coefficients, the other formulations of the product (SIMT
    dequantise-and-FMA kernel, popcount product of two encoded operands, the reference's own CUDA kernels where they
    were built), the M = 2048 prefill GEMM (tensor roofline) and the encoder.  Every timing cycles through more weights
    than L2 holds and is the median of five measurements."""
    import sbvr
    peak, _ = measured_peak()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf_peak = float(json.load(f)["bf16_tflops"])
    except Exception:
        tf_peak = 1590.0
    gen = torch.Generator(device=dev).manual_seed(11)
    shapes = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]

    def mk(N, K, s=S, g=G, direct=False):
        bvr = torch.randint(-2**31, 2**31 - 1, (K // 32, N, s), dtype=torch.int32, device=dev, generator=gen)
        if direct:
            coeff = (torch.randn((K // g, N, s), device=dev, generator=gen) * 0.01).half()
            return sbvr.sbvr.from_packed(bvr, None, coeff, group_len=g, device=dev)
        idx = torch.randint(0, C, (K // g, N), device=dev, generator=gen).to(torch.int16).view(torch.uint16)
        cache = (torch.randn((C, s), device=dev, generator=gen) * 0.01).half()
        return sbvr.sbvr.from_packed(bvr, idx, cache, group_len=g, device=dev)

    def row(N, K, M, s, g, us, ib, algo=None):
        byt = alg_bytes(M, N, K, s=s, g=g, ib=ib, c=(C if ib else 0)) if ib else \
            N * K * s // 8 + N * (K // g) * s * 2 + M * K * 2 + M * N * 2
        gbs = byt / us / 1e3
        r = {"N": N, "K": K, "M": M, "S": s, "G": g, "us": round(us, 2), "GBps": round(gbs, 1), "frac": round(gbs / peak, 4)}
        if algo is not None:
            r["algo"] = algo
        return r

    sweep, prefill, rowdeq, direct128, others, batch = [], [], [], [], [], []
    for N, K in shapes:
        for s in (4, 3, 2):
            ncopy = int(2 * 126e6 / (N * K * s / 8)) + 2
            ws_ = [mk(N, K, s=s) for _ in range(ncopy)]
            for M in ((1, 4, 16, 32) if s == 4 else (1, 16)):
                x = torch.randn((M, K), device=dev, generator=gen).half()
                outs = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(ncopy)]
                us = median_graph_time_us(torch, stream, [(lambda w=w, o=o: sbvr.linear(x, w, None, out=o)) for w, o in zip(ws_, outs)])
                sweep.append(row(N, K, M, s, G, us, IDXB))
            if s == 4:
                # the two kernels for small batches side by side, whatever the automatic choice is
                for M in (16, 32):
                    x = torch.randn((M, K), device=dev, generator=gen).half()
                    outs = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(ncopy)]
                    for algo, name in ((3, "fp16 GEMM with in-kernel dequantisation (linear_gemm_kernel)"),
                                       (4, "FP4 digits with block scale factors (xq8_kernel + linear_tcb_kernel)")):
                        us = median_graph_time_us(torch, stream, [(lambda w=w, o=o: sbvr.linear(x, w, None, algo=algo, out=o))
                                                                  for w, o in zip(ws_, outs)], repeats=3)
                        batch.append(dict(row(N, K, M, 4, G, us, IDXB, algo=algo), kernel=name))
                x = torch.randn((1, K), device=dev, generator=gen).half()
                outs = [torch.empty((1, N), dtype=torch.float16, device=dev) for _ in range(ncopy)]
                us = median_graph_time_us(torch, stream, [(lambda w=w, o=o: sbvr.linear(x, w, None, algo=1, out=o)) for w, o in zip(ws_, outs)], reps=2, repeats=3)
                others.append(dict(row(N, K, 1, 4, G, us, IDXB, algo=1), kernel="SIMT dequantise-and-FMA (linear_simt_kernel)"))
            if s == 4 and N * K == 14336 * 4096:
                M = 2048
                x = torch.randn((M, K), device=dev, generator=gen).half()
                out = torch.empty((M, N), dtype=torch.float16, device=dev)
                us = median_graph_time_us(torch, stream, [(lambda w=w: sbvr.linear(x, w, None, out=out)) for w in ws_[:4]])
                tf = 2.0 * M * N * K / us / 1e6
                prefill.append({"N": N, "K": K, "M": M, "us": round(us, 1), "TFLOPs": round(tf, 1),
                                "frac_of_measured_bf16_burst": round(tf / tf_peak, 4)})
            del ws_
        # group length 128, one coefficient line per (group, row): the configuration the task sheet words (the reference
        # itself hard-wires 256)
        ncopy = int(2 * 126e6 / (N * K * S / 8)) + 2
        wd_ = [mk(N, K, g=128, direct=True) for _ in range(ncopy)]
        for M in (1, 16):
            x = torch.randn((M, K), device=dev, generator=gen).half()
            outs = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(ncopy)]
            us = median_graph_time_us(torch, stream, [(lambda w=w, o=o: sbvr.linear(x, w, None, out=o)) for w, o in zip(wd_, outs)])
            direct128.append(row(N, K, M, S, 128, us, 0))
        del wd_
        # the same product on the transposed ("row-dequant") encoding: packed W^T, groups along the output dimension
        wt_ = [mk(K, N) for _ in range(ncopy)]
        for M in (1, 4):
            x = torch.randn((M, K), device=dev, generator=gen).half()
            us = median_graph_time_us(torch, stream, [(lambda w=w: sbvr.row_deq_mm_T(x, w)) for w in wt_])
            rowdeq.append(row(N, K, M, S, G, us, IDXB))
        # ... and the reference's own kernel for it, compiled for this GPU, on the same tensors (default stream, no graph)
        try:
            from oracle import ref_cuda
            if ref_cuda.lib() is not None:
                x = torch.randn((1, K), device=dev, generator=gen).half()
                us = sum(ref_cuda.time_row_deq_us(x, w.bvr, w.coeff_idx, w.coeff_cache, reps=3) for w in wt_) / len(wt_)
                others.append(dict(row(N, K, 1, S, G, us, IDXB), kernel="reference cuda_1xtN_rd_WP8_TBW4_NS4 (transposed "
                                   "layout, compiled unchanged for sm_100)"))
        except Exception as e:                                  # the comparator is optional
            others.append({"N": N, "K": K, "kernel": "reference row-dequant kernel", "unavailable": str(e)[:120]})
        del wt_
    # popcount product of two encoded operands (the reference's `_sbvr_mm_T`), one encoded activation row
    for N, K in [(4096, 4096), (14336, 4096)]:
        ncopy = int(2 * 126e6 / (N * K * S / 8)) + 2
        rs_ = [mk(N, K) for _ in range(ncopy)]
        a = mk(1, K)
        us = median_graph_time_us(torch, stream, [(lambda w=w: sbvr.mm_T(a, w)) for w in rs_])
        others.append(dict(row(N, K, 1, S, G, us, IDXB), kernel="popcount product, both operands encoded (popc_mm_kernel)"))
        try:
            from oracle import ref_cuda
            if ref_cuda.lib() is not None:
                us = sum(ref_cuda.time_mm_T_us(a.bvr, a.coeff_idx, a.coeff_cache, w.bvr, w.coeff_idx, w.coeff_cache, reps=5)
                         for w in rs_) / len(rs_)
                others.append(dict(row(N, K, 1, S, G, us, IDXB), kernel="reference cuda_1xtN_sbvr_mm_T (compiled unchanged for sm_100)"))
        except Exception as e:
            others.append({"N": N, "K": K, "kernel": "reference popcount kernel", "unavailable": str(e)[:120]})
        del rs_
    # the encoder: a 4096 x 4096 weight (randn * 0.02, the reference's recipe) to packed form, wall clock including the host walk
    import time
    Wd = (torch.randn((4096, 4096), device=dev, generator=gen) * 0.02).half()
    sbvr.sbvr(Wd[:64], encoder_config={"num_sums": S}, device=dev, verbose_level=0)      # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    we = sbvr.sbvr(Wd, encoder_config={"num_sums": S}, device=dev, verbose_level=0)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    rel = float(((we.decode().float() - Wd.float()) ** 2).mean() / (Wd.float() ** 2).mean())
    enc = {"shape": [4096, 4096], "S": S, "seconds": round(dt, 3), "groups_per_s": round(65536 / dt),
           "relative_mse": round(rel, 5), **we.encoder_stats}
    # a bounded wait that ran out in any of the launches above is reported here (and cleared), not in a later section
    from sbvr import _lib
    timeouts = []
    torch.cuda.synchronize()
    for (d_, st_), ws_obj in list(_lib._workspaces.items()):
        if ws_obj.status(st_) != 0:
            timeouts.append(hex(_lib.lib.sbvr_last_timeout_where()))
    return {"bounded_wait_timeouts": timeouts,
            "small_m_sweep": {"G": G, "index": "u16 codebook C=4096", "rows": sweep},
            "group128_direct": {"rows": direct128},
            "small_batch_kernels": {"rows": batch},
            "other_formulations_m1": others, "prefill_gemm": prefill,
            "row_deq_transposed_layout": {"S": S, "G": G, "rows": rowdeq}, "encoder": enc}


def llama_decode(torch, dev, dist, world, preset, batch, prompt, new_tokens):
    """Tokens/s of greedy decoding (CUDA-graph replay of one step) of the SBVR Llama, tensor parallel over all
    ranks of the job; the prompt is prefilled first and timed separately."""
    from models.sbvr_llama import LlamaConfig, SBVRLlamaForCausalLM
    cfg = LlamaConfig.preset(preset)
    group = dist.group.WORLD if dist else None
    m = SBVRLlamaForCausalLM(cfg, device=dev, tp_group=group, max_batch=batch, max_ctx=prompt + new_tokens + 8)
    m.init_synthetic(7)
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), device=dev, generator=torch.Generator(device=dev).manual_seed(99))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m.prefill(ids)
    torch.cuda.synchronize()
    e0.record()
    nxt = m.prefill(ids)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    def timed_decode():
        m.generate(ids, 4)                             # captures the decode graph
        b = m._act(batch, batch)
        with torch.inference_mode():
            b.ids.copy_(nxt)
            b.positions.fill_(prompt)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        e0.record()
        for _ in range(new_tokens):
            m._graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1)
        if dist:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t[0].item())
        return t_ms
    ms = timed_decode()
    nccl_ms, exchange = None, "none (single GPU)"
    if dist:
        exchange = "NCCL all-reduce"
        fused_ms = None
        pull_ms = None
        if m.enable_fused_allreduce(16):               # same decode with the exchanges over symmetric peer memory
            nccl_ms = ms
            m.set_pushed_allreduce(False)              # one-shot all-reduce kernel: flags, then loads over NVLink
            pull_ms = timed_decode()
            fused_ms, fused_name = pull_ms, "fused one-shot all-reduce + add + RMSNorm over symmetric memory (peer loads)"
            if batch <= 4:                             # decode GEMV: results pushed by its epilogue as tagged packets
                m.set_pushed_allreduce(True)
                push_ms = timed_decode()
                if push_ms <= fused_ms:
                    fused_ms, fused_name = push_ms, ("row-parallel GEMV pushes epoch-tagged packets to every rank, packet "
                                                     "reduce + add + RMSNorm on the receiver (no flags, no peer loads)")
            if fused_ms <= nccl_ms:                    # the fastest exchange is the one reported as tokens_per_s
                ms = fused_ms
                exchange = fused_name
        t = torch.tensor([prefill_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms = float(t[0].item())
    m._check()
    wbytes = m.packed_weight_bytes()
    peak, _ = measured_peak()
    res = {"model": preset, "tp": world, "batch": batch, "prompt": prompt, "new_tokens": new_tokens,
           "tokens_per_s": round(batch * new_tokens / ms * 1e3, 1), "ms_per_step": round(ms / new_tokens, 4),
           "prefill_ms": round(prefill_ms, 2), "packed_weight_bytes_per_gpu": wbytes,
           "weight_stream_GBps_per_gpu": round(wbytes / (ms / new_tokens) / 1e6, 1),
           "frac_of_hbm_roofline": round(wbytes / (ms / new_tokens) / 1e6 / peak, 4), "exchange": exchange}
    if nccl_ms is not None:
        res["tokens_per_s_nccl"] = round(batch * new_tokens / nccl_ms * 1e3, 1)
        res["tokens_per_s_fused_allreduce"] = round(batch * new_tokens / fused_ms * 1e3, 1)
        res["tokens_per_s_one_shot_peer_loads"] = round(batch * new_tokens / pull_ms * 1e3, 1)
        if batch <= 4:
            res["tokens_per_s_pushed_packets"] = round(batch * new_tokens / push_ms * 1e3, 1)
    del m
    torch.cuda.empty_cache()
    return res


def cpu_layer_step(O, np, packed, xs):
    """One STEP of the workload on the CPU port: the seven linears of the layer, each on its own packed weight."""
    for name, N, K in SHAPES:
        p = packed[(N, K)]
        O.linear_c(xs[K], p["bvr"], p["coeff_idx"], p["coeff"], G=G)


def cpu_baseline(steps=None, budget_s=10.0):
    """The CPU port of the reference arithmetic (oracle/sbvr_oracle.c: fused decode + dot with fp32 accumulation, OpenMP over
    output rows; the reference's own native kernels are ARM-NEON code that does not build on this host), timed on this
    host's cores on whole STEPS of the workload: all four layer shapes, seven linears per step.  `steps` fixes the number
    of steps; otherwise steps are run until about `budget_s` seconds have passed."""
    import numpy as np
    from oracle import sbvr_oracle as O
    packed = {(N, K): O.make_packed(N, K, S, G=G, mode="u16", C=C, seed=7 + i) for i, (N, K) in
              enumerate(sorted({(n, k) for _, n, k in SHAPES}))}
    rng = np.random.default_rng(1)
    xs = {K: rng.standard_normal((1, K)).astype(np.float16) for K in {k for _, _, k in SHAPES}}
    O.c_lib().sbvr_oracle_set_threads(os.cpu_count() or 1)      # torchrun exports OMP_NUM_THREADS=1
    threads = O.c_lib().sbvr_oracle_threads()
    cpu_layer_step(O, np, packed, xs)                            # warm-up
    t0 = time.perf_counter()
    n = 0
    while True:
        cpu_layer_step(O, np, packed, xs)
        n += 1
        el = time.perf_counter() - t0
        if (steps and n >= steps) or (not steps and (el > budget_s or n >= 1000)):
            break
    gbs = STEP_BYTES * n / el / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{n} whole steps (7 SBVR linears of the layer: 4096x4096 x2, 1024x4096 x2, 14336x4096 x2, "
                      f"4096x14336; S=4 G=256 M=1), {el / n * 1e3:.2f} ms per step",
            "ms_per_step": round(el / n * 1e3, 3)}


def run_reference(args):
    """The reference's own way of running this path on a CPU is `x @ decode().T` (its native kernels are ARM-NEON only and
    take encoded activations); the C port of that arithmetic is what can run here.  Same workload, metric and unit as the
    GPU arm: whole steps of the seven layer linears, all host threads."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    t_all = time.perf_counter()
    steps = max(1, min(args.steps, 300))                         # 300 steps are about 20 s of CPU work
    base = cpu_baseline(steps=steps)
    v = base["value"]
    line = {"metric": "sbvr_gemv_hbm_gbs_m1", "value": v, "unit": "GB/s", "impl": "reference",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama3-8b decoder-layer linears (q,k,v,o,gate,up,down), M=1, S=4, G=256, "
                                   "u16 codebook C=4096", "bytes_per_step": STEP_BYTES,
                       "note": f"CPU port of the reference arithmetic on all host threads; {steps} whole steps timed "
                               "(bounded at 300)"},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": round(time.perf_counter() - t_all, 1)}
    print(json.dumps(line), flush=True)


def decode_step_case():
    """One eager decode step (batch 1, context 512) of a 4-layer model with Llama-3-8B layer shapes, inside the NVTX
    range "decode", after a prefill and two warm-up steps."""
    import torch
    from models.sbvr_llama import LlamaConfig, SBVRLlamaForCausalLM
    cfg = LlamaConfig.preset("8b")
    cfg.num_hidden_layers = 4
    m = SBVRLlamaForCausalLM(cfg, max_batch=1, max_ctx=600).init_synthetic(7)
    ids = torch.randint(0, cfg.vocab_size, (1, 512), device="cuda", generator=torch.Generator(device="cuda").manual_seed(99))
    nxt = m.prefill(ids)
    pos = torch.full((1,), 512, dtype=torch.int32, device="cuda")
    for _ in range(2):
        m.decode_step(nxt, pos)
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push("decode")
    m.decode_step(nxt, pos)
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    print(json.dumps({"kernel_case": "decode_step", "layers": 4, "context": 512}))


def kernel_case(which):
    """Six 14336 x 4096 weights (176 MB, more than L2), two warm-up rounds, then one launch per weight."""
    if which == "decode_step":
        return decode_step_case()
    import torch
    import sbvr
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(7)
    N, K = 14336, 4096
    if which == "rowdeq":
        # the transposed encoding: packed W^T, i.e. a [K rows, N along the bits] matrix in the same layout
        wt_ = []
        for _ in range(6):
            bvr = torch.randint(-2**31, 2**31 - 1, (N // 32, K, S), dtype=torch.int32, device=dev, generator=gen)
            idx = torch.randint(0, C, (N // G, K), device=dev, generator=gen).to(torch.int16).view(torch.uint16)
            cache = (torch.randn((C, S), device=dev, generator=gen) * 0.01).half()
            wt_.append(sbvr.sbvr.from_packed(bvr, idx, cache, group_len=G, device=dev))
        x = torch.randn((1, K), device=dev, generator=gen).half()
        for _ in range(3):
            for w in wt_:
                y = sbvr.row_deq_mm_T(x, w)
        torch.cuda.synchronize()
        print(json.dumps({"kernel_case": which, "launches": 18, "mean_abs_y": float(y.float().abs().mean())}))
        return
    if which == "encode":
        W = (torch.randn((1024, 4096), device=dev, generator=gen) * 0.02).half()
        w = sbvr.sbvr(W, encoder_config={"num_sums": S}, device=dev, verbose_level=0)
        print(json.dumps({"kernel_case": which, **w.encoder_stats}))
        return
    M = {"gemv": 1, "gemm16": 16, "batch16": 16, "gemm2048": 2048}[which]
    algo = {"gemm16": 3, "batch16": 4}.get(which, 0)      # M = 16: the fp16 GEMM or the small-batch FP4 kernel on request
    ws_ = []
    for _ in range(6):
        bvr = torch.randint(-2**31, 2**31 - 1, (K // 32, N, S), dtype=torch.int32, device=dev, generator=gen)
        idx = torch.randint(0, C, (K // G, N), device=dev, generator=gen).to(torch.int16).view(torch.uint16)
        cache = (torch.randn((C, S), device=dev, generator=gen) * 0.01).half()
        ws_.append(sbvr.sbvr.from_packed(bvr, idx, cache, group_len=G, device=dev))
    x = torch.randn((M, K), device=dev, generator=gen).half()
    y = torch.empty((M, N), dtype=torch.float16, device=dev)
    for _ in range(3):
        for w in ws_:
            sbvr.linear(x, w, None, algo=algo, out=y)
    torch.cuda.synchronize()
    print(json.dumps({"kernel_case": which, "launches": 18, "mean_abs_y": float(y.float().abs().mean())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline GEMV measurement (no M sweep, prefill GEMM or Llama decode sections)")
    ap.add_argument("--skip-70b", action="store_true", help="leave the 70B decode out of the Llama section")
    ap.add_argument("--kernel-case", default=None, choices=["gemv", "gemm16", "batch16", "gemm2048", "decode_step", "rowdeq", "encode"],
                    help="run a few launches of one kernel on 14336x4096 weights, or one eager decode step of a "
                         "4-layer Llama-3-8B-shaped model inside the NVTX range 'decode', and exit (for profilers)")
    args = ap.parse_args()
    if args.kernel_case:
        return kernel_case(args.kernel_case)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
