"""Builds an `SBVRLlamaForCausalLM` from a directory of per-projection files as the reference's encoder writes them.

Directory convention (reference encode_llama.py:19-33, :42-50; sbvr_utils/utils_llama.py:132-158):
    layer_{i}_{q,k,v,gate_proj,up_proj,down_proj}.pt     one `sbvr.save` file per projection
    lm_head_weight.pt                                    optional
The reference never encodes o_proj (its flow decodes every file back to dense fp16 and leaves o_proj as it was), so
o_proj -- like the embedding and the norm weights -- comes from the dense state dict of the checkpoint; a file
`layer_{i}_o.pt` is used when present.  Nothing is decoded here: the packed tensors are sliced for the rank, fused
(q|k|v, gate|up) and handed to `SBVRLinear`.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

import sbvr as _sbvr

from . import parallel
from .sbvr_llama import SBVRLinear, SBVRLlamaDecoderLayer, SBVRLlamaForCausalLM

ATTN = ("q", "k", "v")
FFN = ("gate_proj", "up_proj", "down_proj")


class DenseLinear(torch.nn.Module):
    """A projection the checkpoint holds as dense fp16 (o_proj in reference-encoded directories): a plain library
    GEMM, same call form as `SBVRLinear`."""

    def __init__(self, weight: torch.Tensor):
        super().__init__()
        self.weight_dense = weight.contiguous()
        self.in_features, self.out_features = weight.shape[1], weight.shape[0]

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return torch.matmul(x, self.weight_dense.t(), out=out)

    def packed_bytes(self) -> int:
        return self.weight_dense.numel() * 2


def read_packed(path: str, device) -> dict:
    """One `sbvr.save` file -> {"bvr", "coeff_idx", "coeff_cache", "group_len"} on `device` (tensors as stored)."""
    w = _sbvr.load(path, device=torch.device(device), verbose_level=0)
    return {"bvr": w.bvr.view(torch.int32), "coeff_idx": w.coeff_idx, "coeff_cache": w.coeff_cache,
            "group_len": w.bvr_len, "shape": tuple(w.original_data_shape)}


def read_layer(weight_dir: str, i: int, device) -> Dict[str, dict]:
    out = {}
    for name in ATTN + FFN + ("o",):
        path = os.path.join(weight_dir, f"layer_{i}_{name}.pt")
        if os.path.exists(path):
            out[name] = read_packed(path, device)
        elif name != "o":
            raise FileNotFoundError(path)
    return out


def _linear(p: dict, device) -> SBVRLinear:
    w = _sbvr.sbvr.from_packed(p["bvr"], p["coeff_idx"], p["coeff_cache"], group_len=p.get("group_len", 256),
                               device=torch.device(device))
    return SBVRLinear.from_sbvr(w)


@torch.inference_mode()
def load_directory(model: SBVRLlamaForCausalLM, weight_dir: str, dense_state: Dict[str, torch.Tensor]):
    """Fills `model` (already constructed with its config, device and tensor-parallel group) from `weight_dir` and
    the checkpoint's dense tensors (HuggingFace names: model.embed_tokens.weight, model.layers.{i}.*, model.norm.weight,
    lm_head.weight)."""
    c, dev, r, n = model.config, model.device, model.tp_rank, model.tp_size
    f16 = lambda t: t.to(device=dev, dtype=torch.float16).contiguous()
    model.embed_tokens = f16(dense_state["model.embed_tokens.weight"])
    model.layers = []
    for i in range(c.num_hidden_layers):
        L = read_layer(weight_dir, i, dev)
        G = L["q"]["group_len"]
        qkv = parallel.fuse_rows([parallel.shard_rows(L[k], r, n) for k in ATTN])
        gu = parallel.fuse_rows([parallel.shard_rows(L["gate_proj"], r, n), parallel.shard_rows(L["up_proj"], r, n)])
        qkv["group_len"] = gu["group_len"] = G
        down = parallel.shard_cols(L["down_proj"], r, n, G)
        down["group_len"] = G
        if "o" in L:
            o_p = parallel.shard_cols(L["o"], r, n, G)
            o_p["group_len"] = G
            o = _linear(o_p, dev)
        else:
            W = dense_state[f"model.layers.{i}.self_attn.o_proj.weight"]
            k0, k1 = r * W.shape[1] // n, (r + 1) * W.shape[1] // n
            o = DenseLinear(f16(W[:, k0:k1]))
        model.layers.append(SBVRLlamaDecoderLayer(
            _linear(qkv, dev), o, _linear(gu, dev), _linear(down, dev),
            f16(dense_state[f"model.layers.{i}.input_layernorm.weight"]),
            f16(dense_state[f"model.layers.{i}.post_attention_layernorm.weight"])))
    model.norm_weight = f16(dense_state["model.norm.weight"])
    head_path = os.path.join(weight_dir, "lm_head_weight.pt")
    if os.path.exists(head_path):
        hp = parallel.shard_rows(read_packed(head_path, dev), r, n)
        model.lm_head = _linear(hp, dev)
    else:
        W = dense_state["lm_head.weight"]
        v0, v1 = r * W.shape[0] // n, (r + 1) * W.shape[0] // n
        model.lm_head = DenseLinear(f16(W[v0:v1]))
    model._alloc_cache()
    return model
