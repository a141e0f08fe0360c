"""Host-side checks that need no GPU: the C-ABI library loads and exports what the header declares,
argument validation, the tile partition of the persistent grid, the serialized file format."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import sbvr
    from sbvr import _lib
    hdr = open(os.path.join(ROOT, "include", "sbvr_b200.h")).read()
    declared = re.findall(r"SBVR_API\s+[\w\s\*]+?\b(sbvr_\w+)\s*\(", hdr)
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(_lib.lib, name), name
    assert set(declared) == set(_lib.EXPORTS)
    assert {"sbvr", "_sbvr_serialized", "load", "mm_T", "linear"} <= set(dir(sbvr))


def test_strerror_and_validation_without_gpu():
    from sbvr import _lib
    L = _lib.lib
    assert _lib.strerror(0) == "ok"
    for rc in range(-7, 0):
        assert "unknown" not in _lib.strerror(rc)
    buf = (ctypes.c_uint32 * 64)()
    p = ctypes.addressof(buf)
    # null pointers, bad S, bad G, K % G, idx/C mismatch: all rejected before any CUDA call
    assert L.sbvr_linear_f16(None, p, p, 1, p, 4, None, p, 1, 64, 256, 4, 256, 0, None, None) == -1
    assert L.sbvr_linear_f16(p, p, p, 1, p, 4, None, p, 1, 64, 256, 9, 256, 0, None, None) == -1
    assert L.sbvr_linear_f16(p, p, p, 1, p, 4, None, p, 1, 64, 256, 4, 100, 0, None, None) == -1
    assert L.sbvr_linear_f16(p, p, p, 1, p, 4, None, p, 1, 64, 300, 4, 256, 0, None, None) == -2
    assert L.sbvr_linear_f16(p, p, p, 1, p, 300, None, p, 1, 64, 256, 4, 256, 0, None, None) == -1
    assert L.sbvr_linear_f16(p, p, p, 3, p, 4, None, p, 1, 64, 256, 4, 256, 0, None, None) == -1
    assert L.sbvr_linear_f16(p, p + 1, p, 1, p, 4, None, p, 1, 64, 256, 4, 256, 0, None, None) == -3
    assert L.sbvr_decode_f16(p, p, 1, p, 4, None, 256, 64, 256, 256, 4, 256, None) == -1
    assert L.sbvr_decode_f16(p, p, 1, p, 4, p, 100, 64, 256, 256, 4, 256, None) == -1     # ldw < K_out
    assert L.sbvr_workspace_status(None, None) == -1


def test_reference_written_file_loads(golden):
    """A file saved by the reference's `sbvr.save` unpickles into this package's classes."""
    import sbvr
    path = os.path.join(ROOT, "tests", "golden", "ser_enc_s4.pt")
    w = sbvr.load(path, device=torch.device("cpu"), verbose_level=0)
    c = golden["enc_s4"]
    assert w.num_sums == 4 and w.bvr_len == 256
    assert tuple(w.original_data_shape) == (8, 512)
    assert np.array_equal(w.bvr.view(torch.int32).numpy().view(np.uint32), c["bvr"])
    assert np.array_equal(w.coeff_idx.numpy(), c["coeff_idx"])
    assert np.array_equal(w.coeff_cache.numpy().view(np.uint16), c["coeff_cache"].view(np.uint16))


def test_save_load_roundtrip(tmp_path, golden):
    import sbvr
    c = golden["syn_u16_s3"]
    w = sbvr.sbvr.from_packed(torch.from_numpy(c["bvr"].view(np.int32)),
                              torch.from_numpy(c["coeff_idx"].view(np.int16)).view(torch.uint16),
                              torch.from_numpy(c["coeff_cache"]), device=torch.device("cpu"))
    f = str(tmp_path / "w.pt")
    w.save(f)
    w2 = sbvr.load(f, device=torch.device("cpu"), verbose_level=0)
    assert torch.equal(w2.bvr.view(torch.int32), w.bvr.view(torch.int32))
    assert torch.equal(w2.coeff_idx.view(torch.int16), w.coeff_idx.view(torch.int16))
    assert torch.equal(w2.coeff_cache, w.coeff_cache)
    assert w2.num_sums == 3


def test_constructor_errors_match_reference():
    import sbvr
    with pytest.raises(ValueError):
        sbvr.sbvr()
    with pytest.raises(ValueError):
        sbvr.sbvr(sbvr_serialized=object())
    with pytest.raises(ValueError):
        sbvr.sbvr.from_packed(torch.zeros((8, 4, 2), dtype=torch.int32), torch.zeros((1, 4), dtype=torch.uint16),
                              torch.zeros((4, 2), dtype=torch.float16), device=torch.device("cpu"))


def test_no_cpu_fallback():
    """Without a CUDA device the product path must refuse, not compute somewhere else."""
    import sbvr
    w = sbvr.sbvr.from_packed(torch.zeros((8, 64, 2), dtype=torch.int32), torch.zeros((1, 64), dtype=torch.uint8),
                              torch.zeros((4, 2), dtype=torch.float16), device=torch.device("cpu"))
    with pytest.raises(RuntimeError):
        sbvr.linear(torch.zeros((1, 256), dtype=torch.float16), w)
    with pytest.raises(RuntimeError):
        w.decode()


def test_glue_and_fused_entry_points_validate_before_any_cuda_call():
    from sbvr import _lib
    L = _lib.lib
    buf = (ctypes.c_uint32 * 64)()
    p = ctypes.addressof(buf)
    assert L.sbvr_add_rmsnorm_f16(None, None, p, None, p, 1, 4096, 1e-5, None) == -1
    assert L.sbvr_add_rmsnorm_f16(p, None, p, None, p, 1, 4100, 1e-5, None) == -2          # hidden % 8
    assert L.sbvr_add_rmsnorm_f16(p + 2, None, p, None, p, 1, 4096, 1e-5, None) == -3      # alignment
    assert L.sbvr_rope_append_f16(p, p, p, 1.0, p, p, 3, 2, 4, 2, 128, 64, None) == -1     # tokens % tokens_per_seq
    assert L.sbvr_attention_f16(p, p, p, p, p, None, 1, 1, 6, 4, 128, 64, 0.1, 1, None) == -1   # heads % kv heads
    assert L.sbvr_attention_f16(p, p, p, p, p, None, 1, 1, 4, 2, 64, 64, 0.1, 1, None) == -7    # head_dim
    assert L.sbvr_attention_f16(p, p, p, p, p, None, 1, 1, 4, 2, 128, 64, 0.1, 4, None) == -5   # splits need scratch
    assert L.sbvr_rope_attention_f16(p, p, None, 1.0, p, p, p, None, 1, 4, 2, 128, 64, 0.1, 1, None) == -1
    assert L.sbvr_silu_mul_f16(p, p, 1, 12, None) == -2
    assert L.sbvr_embedding_f16(None, p, p, 1, 64, None) == -1
    assert L.sbvr_argmax_f16(p, None, None, 1, 10, None) == -1
    # fused linear: unknown op, bad packed arguments, missing workspace
    assert L.sbvr_linear_fused_f16(7, p, None, None, None, 0.0, p, p, 1, p, 4, None, p, 1, 64, 256, 4, 256, None, None) == -1
    assert L.sbvr_linear_fused_f16(1, p, None, None, None, 0.0, p, p, 1, p, 4, None, p, 1, 64, 300, 4, 256, None, None) == -2
    assert L.sbvr_linear_fused_f16(1, p, None, None, None, 0.0, p, p, 1, p, 4, None, p, 1, 64, 256, 4, 256, None, None) == -5
    assert L.sbvr_allreduce_add_rmsnorm_f16(p, p, p, 3, 0, 0, 2, 4096, p, p, p, p, 1, 4096, 1e-5, None, None) == -1
    out = ctypes.c_size_t(0)
    assert L.sbvr_workspace_bytes(0, 0, 64, 256, ctypes.byref(out)) == -1


def test_encoder_config_and_search_space_on_cpu():
    """Host side of the encoder: unknown keys are ignored, unsupported settings are refused, and the candidate lines of a
    group have the reference's counts (r x b x s lists plus the plain grid; sbvr/core.py:400-483) and are sorted by
    magnitude inside each line."""
    import pytest
    import torch
    from sbvr import encoder
    conf = encoder.EncoderConfig.from_dict({"num_sums": 3, "verbose": 1})
    assert conf.num_sums == 3 and conf.r_search_num == 64
    with pytest.raises(ValueError):
        encoder.EncoderConfig.from_dict({"num_sums": 5})
    with pytest.raises(ValueError):
        encoder.EncoderConfig.from_dict({"error_function": "input_inner"})
    g = torch.Generator().manual_seed(0)
    d = (torch.randn(256, generator=g) * 0.02).half()
    space = encoder.group_search_space(d, encoder.EncoderConfig(num_sums=4, space_device="cpu"), False)
    assert space.dtype == torch.float16 and space.shape == (64 * 40 * 40 + 20 ** 4, 4)
    a = space.abs().float()
    assert bool((a[:, 1:] >= a[:, :-1]).all())
    with pytest.raises(RuntimeError):
        encoder.encode(d.view(1, -1), encoder.EncoderConfig(), device=torch.device("cpu"))


def test_step_partition_of_the_streaming_kernels(tmp_path):
    """The split of (tile, k step) work over the CTAs that the decode GEMV and the small-batch kernel share (TsSegs in
    csrc/tc_stream.cuh) is compiled for the host and checked over a few thousand (tiles, steps, CTAs) combinations: every
    step owned once, shared segments first and at most two per CTA, owners of the left-over steps as cta_of() says."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    exe = str(tmp_path / "partition_check")
    src = os.path.join(ROOT, "tests", "native", "partition_check.cu")
    subprocess.check_call([nvcc, "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
                           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "sbvr-cpu-arm_b200", "csrc"),
                           "-o", exe, src])
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:]
    assert "0 failures" in out.stdout
