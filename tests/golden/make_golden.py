"""Generate the golden vectors in this directory by running the reference's own code.

Run once, in a container where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `sbvr/core.py` by file path (the `sbvr` package itself
cannot be imported on x86: its `__init__` loads ARM-NEON extensions) and stores,
per case, the packed tensors and what the reference computes from them:

  enc_*   weights `randn * 0.02` pushed through the reference ENCODER
          (`sbvr(data, {"num_sums": S})`), then `decode()`, then the reference
          product `x @ decode().T + bias` in fp16 on CPU (test_sbvr.py:321).
  syn_*   seeded Bernoulli(0.5) planes + random codebook wrapped in the
          reference's `_sbvr_serialized`, loaded with `sbvr(sbvr_serialized=…)`,
          then `decode()` and the same product.
  ser_*   one `save()`d file (the reference's pickle of `_sbvr_serialized`),
          to pin the on-disk format.

The files are small `.npz` archives; nothing at test time reads the reference.
"""
import importlib.util
import io
import os
import sys
import contextlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import sbvr_oracle as O  # noqa: E402


def load_reference(ref_root):
    # registered as `sbvr.core` under a stand-in parent package so that the pickle written by
    # `save()` names the class `sbvr.core._sbvr_serialized`, exactly as a reference install would
    import types
    spec = importlib.util.spec_from_file_location("sbvr.core", os.path.join(ref_root, "sbvr", "core.py"))
    mod = importlib.util.module_from_spec(spec)
    pkg = types.ModuleType("sbvr")
    pkg.__path__ = []
    pkg.core = mod
    sys.modules["sbvr"] = pkg
    sys.modules["sbvr.core"] = mod
    spec.loader.exec_module(mod)
    return mod


def t2n(t):
    t = t.detach().cpu()
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32).copy()
    if t.dtype == torch.uint16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def product(ref_w, x, bias):
    dec = ref_w.decode()
    y = x @ dec.T
    if bias is not None:
        y = y + bias
    return dec, y


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SBVR_REFERENCE_DIR", "")
    if not ref_root:
        sys.exit("usage: make_golden.py <path of a checkout of the reference>  (or SBVR_REFERENCE_DIR)")
    core = load_reference(ref_root)
    cpu = torch.device("cpu")
    out = {}

    # ---- encoder cases ---------------------------------------------------
    enc_cases = [("enc_s2", 8, 512, 2, 3), ("enc_s3", 8, 512, 3, 4), ("enc_s4", 8, 512, 4, 5),
                 ("enc_s4_pad", 6, 300, 4, 6)]
    for name, N, K, S, seed in enc_cases:
        g = torch.Generator().manual_seed(seed)
        W = (torch.randn((N, K), generator=g) * 0.02).to(torch.float16)
        x = torch.randn((3, K), generator=g).to(torch.float16)
        bias = (torch.randn((N,), generator=g) * 0.3).to(torch.float16)
        with contextlib.redirect_stdout(io.StringIO()):
            w = core.sbvr(W, encoder_config={"num_sums": S}, device=cpu, verbose_level=-1)
        dec, y = product(w, x, bias)
        _, y_nobias = product(w, x, None)
        case = dict(W=t2n(W), x=t2n(x), bias=t2n(bias), bvr=t2n(w.bvr), coeff_idx=t2n(w.coeff_idx),
                    coeff_cache=t2n(w.coeff_cache), decoded=t2n(dec), y=t2n(y), y_nobias=t2n(y_nobias),
                    S=np.int64(S), G=np.int64(w.bvr_len), K=np.int64(K), N=np.int64(N))
        # the numpy restatement must agree with the reference bit for bit
        mine = O.decode(case["bvr"], case["coeff_idx"], case["coeff_cache"], G=256, K=K)
        assert np.array_equal(mine.view(np.uint16), case["decoded"].view(np.uint16)), name
        for k, v in case.items():
            out[f"{name}/{k}"] = v
        print(name, "C =", w.coeff_cache.shape[0], "idx dtype", w.coeff_idx.dtype, "ok")
        if name == "enc_s4":
            path = os.path.join(HERE, "ser_enc_s4.pt")
            w.verbose_level = 0
            w.save(path)

    # ---- synthetic packed tensors through the reference loader + decoder ----
    syn_cases = [("syn_u8_s4", 32, 1024, 4, "u8", 200), ("syn_u16_s4", 32, 1024, 4, "u16", 700),
                 ("syn_u8_s2", 16, 512, 2, "u8", 256), ("syn_u16_s3", 16, 768, 3, "u16", 300),
                 ("syn_u8_s6", 8, 512, 6, "u8", 17), ("syn_u16_s8", 8, 256, 8, "u16", 1000)]
    for i, (name, N, K, S, mode, C) in enumerate(syn_cases):
        p = O.make_packed(N, K, S, G=256, mode=mode, C=C, seed=100 + i)
        bvr_t = torch.from_numpy(p["bvr"].view(np.int32)).view(torch.uint32)
        if mode == "u8":
            idx_t = torch.from_numpy(p["coeff_idx"])
        else:
            idx_t = torch.from_numpy(p["coeff_idx"].view(np.int16)).view(torch.uint16)
        cache_t = torch.from_numpy(p["coeff"])
        ser = core._sbvr_serialized(S, 256, torch.float16, torch.uint32, torch.float16, torch.Size((N, K)),
                                    bvr_t, idx_t, cache_t, -1, None)
        w = core.sbvr(sbvr_serialized=ser, device=cpu, verbose_level=0)
        g = torch.Generator().manual_seed(1000 + i)
        x = torch.randn((2, K), generator=g).to(torch.float16)
        bias = (torch.randn((N,), generator=g) * 0.3).to(torch.float16)
        dec, y = product(w, x, bias)
        case = dict(x=t2n(x), bias=t2n(bias), bvr=p["bvr"], coeff_idx=p["coeff_idx"], coeff_cache=p["coeff"],
                    decoded=t2n(dec), y=t2n(y), S=np.int64(S), G=np.int64(256), K=np.int64(K), N=np.int64(N))
        mine = O.decode(case["bvr"], case["coeff_idx"], case["coeff_cache"], G=256, K=K)
        assert np.array_equal(mine.view(np.uint16), case["decoded"].view(np.uint16)), name
        for k, v in case.items():
            out[f"{name}/{k}"] = v
        print(name, "ok")

    np.savez_compressed(os.path.join(HERE, "sbvr_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "sbvr_golden.npz"))


if __name__ == "__main__":
    main()
