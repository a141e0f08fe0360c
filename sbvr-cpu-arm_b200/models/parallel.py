"""Slicing and fusing of packed SBVR weights: tensor-parallel shards and fused projections.

A packed weight is a dict of `bvr` int32/uint32 [K/32, N, S], `coeff_idx` uint8|uint16 [K/G, N] and
`coeff_cache` fp16 [C, S] (reference layout, sbvr/core.py:724-805).  Output rows are dimension 1 of `bvr` and
`coeff_idx`; input columns are dimension 0 (32 per word, G per index row), so both kinds of shard are plain
slices and need no re-encoding.  Pure tensor indexing: runs on CPU and GPU alike.
"""
from __future__ import annotations

from typing import List

import torch


def shard_rows(p: dict, rank: int, world: int) -> dict:
    """Column-parallel shard (q, k, v, gate, up, lm_head): output rows [rank N/world, (rank+1) N/world)."""
    N = p["bvr"].shape[1]
    if N % world:
        raise ValueError(f"{N} output rows do not divide over {world} ranks")
    n0, n1 = rank * (N // world), (rank + 1) * (N // world)
    return {"bvr": p["bvr"][:, n0:n1, :].contiguous(), "coeff_idx": p["coeff_idx"][:, n0:n1].contiguous(),
            "coeff_cache": p["coeff_cache"]}


def shard_cols(p: dict, rank: int, world: int, group_len: int = 256) -> dict:
    """Row-parallel shard (o, down): input columns [rank K/world, (rank+1) K/world); the shard boundary must fall on
    a group boundary.  The partial products of the ranks are summed by an all-reduce."""
    K = p["bvr"].shape[0] * 32
    if K % (world * group_len):
        raise ValueError(f"{K} input columns do not divide over {world} ranks in groups of {group_len}")
    k0, k1 = rank * (K // world), (rank + 1) * (K // world)
    return {"bvr": p["bvr"][k0 // 32:k1 // 32].contiguous(),
            "coeff_idx": p["coeff_idx"][k0 // group_len:k1 // group_len].contiguous(),
            "coeff_cache": p["coeff_cache"]}


def _idx_as_int(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.uint8:
        return t.to(torch.int32)
    return t.view(torch.int16).to(torch.int32) & 0xFFFF


def fuse_rows(parts: List[dict]) -> dict:
    """Stacks projections that read the same input (q|k|v, gate|up) into one weight with the rows concatenated.
    Equal codebooks are kept once; different ones are concatenated and the indices shifted."""
    caches, offsets, total = [], [], 0
    for p in parts:
        c = p["coeff_cache"]
        hit = None
        for j, prev in enumerate(caches):
            if prev.shape == c.shape and (prev is c or torch.equal(prev, c)):
                hit = j
                break
        if hit is None:
            caches.append(c)
            offsets.append(total)
            total += c.shape[0]
        else:
            offsets.append(sum(x.shape[0] for x in caches[:hit]))
    if total > 65536:
        raise ValueError("fused codebook exceeds 65536 lines")
    idx = torch.cat([_idx_as_int(p["coeff_idx"]) + off for p, off in zip(parts, offsets)], dim=1)
    idx = idx.to(torch.uint8) if total <= 256 else idx.to(torch.int16).view(torch.uint16)
    return {"bvr": torch.cat([p["bvr"] for p in parts], dim=1).contiguous(), "coeff_idx": idx.contiguous(),
            "coeff_cache": torch.cat(caches, dim=0).contiguous()}
