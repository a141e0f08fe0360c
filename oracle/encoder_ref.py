"""CPU restatement of the reference ENCODER's decisions, group by group, for the parity tests.  TEST INFRASTRUCTURE ONLY:
nothing in the package imports this file.

It follows `_encode_to_sbvr` / `_encode_data` / `_search_coeff_bias_space` / `_data_diff_min_mse`
(sbvr/core.py:655-722, :555-653, :529-553, :485-500) literally: one group at a time, the squared differences to every
candidate materialised as fp16 tensors (in chunks), fp16 minimum over the 2^S sums, fp32 mean, first minimum wins.
The candidate lines of a group come from a generator passed in by the caller (the tests pass the package's
`group_search_space`, which is compared with the reference's own generator when the golden vectors are made), so that
this file pins the walk and the error function independently of the CUDA kernels.

Pinned: `tests/test_oracle.py` reproduces the reference encoder's packed output of a golden case bit for bit.
"""
from __future__ import annotations

import itertools
from typing import Callable, List, Optional, Tuple

import numpy as np
import torch

GROUP = 256


def bin_combs(S: int) -> torch.Tensor:
    """Rows of 0/1, first column = most significant selector bit (sbvr/core.py:345-351)."""
    return torch.tensor(list(itertools.product([0, 1], repeat=S)), dtype=torch.float16)


def min_mse(data: torch.Tensor, lines: torch.Tensor, chunk: int = 4096) -> Tuple[float, int, torch.Tensor]:
    """(mse, index, selectors) of the best line for one group (`_get_min_mse_coeff` + `_data_diff_min_mse`,
    sbvr/core.py:520-527, :485-500).  data fp16 [256], lines fp16 [n, S]."""
    S = lines.shape[1]
    combs = bin_combs(S)
    best = (float("inf"), -1, None)
    d = data.view(1, -1, 1)
    for c0 in range(0, lines.shape[0], chunk):
        pts = lines[c0:c0 + chunk] @ combs.T                               # fp16 [c, 2^S]
        diff = (d - pts.view(pts.shape[0], 1, pts.shape[1])) ** 2          # fp16 [c, 256, 2^S]
        picked, sel = diff.min(dim=-1)
        mse = picked.to(torch.float32).mean(dim=-1)
        at = int(mse.argmin())
        if float(mse[at]) < best[0]:                                       # strict: the first of equal minima stays
            best = (float(mse[at]), c0 + at, sel[at].clone())
    return best


def mse_table(data: torch.Tensor, lines: torch.Tensor) -> np.ndarray:
    """fp32 [groups, n]: the MSE of every group against every line (what `sbvr_encode_mse_f16` returns)."""
    combs = bin_combs(lines.shape[1])
    pts = lines @ combs.T
    out = np.empty((data.shape[0], lines.shape[0]), dtype=np.float32)
    for b in range(data.shape[0]):
        diff = (data[b].view(1, -1, 1) - pts.view(pts.shape[0], 1, pts.shape[1])) ** 2
        out[b] = diff.min(dim=-1)[0].to(torch.float32).mean(dim=-1).numpy()
    return out


def selectors(data: torch.Tensor, line: torch.Tensor) -> np.ndarray:
    """uint8 [256]: index of the nearest of the 2^S sums of `line` for every value (first on ties)."""
    pts = (line.view(1, -1) @ bin_combs(line.shape[0]).T).view(-1)
    diff = (data.view(-1, 1) - pts.view(1, -1)) ** 2
    return diff.min(dim=-1)[1].to(torch.uint8).numpy()


def encode(W: torch.Tensor, S: int, space_of: Callable[[torch.Tensor, bool], torch.Tensor], warmup: int = 10,
           window: int = 20, acceptable: float = 10 ** -12, max_lines: int = 2 ** 16, max_groups: Optional[int] = None):
    """Sequential walk over the groups of W (fp16 [N, K]) -> dict(sel uint8 [groups, 256], line_of, lines fp16 [C, S]).
    `space_of(group, extended)` returns the candidate lines of a group.  `max_groups` stops early (prefix check)."""
    N, K = W.shape
    Kp = (K + GROUP - 1) // GROUP * GROUP
    Wp = torch.zeros((N, Kp), dtype=torch.float16)
    Wp[:, :K] = W
    groups = Wp.view(-1, GROUP)
    NG = groups.shape[0] if max_groups is None else min(max_groups, groups.shape[0])
    lines = torch.zeros((max_lines, S), dtype=torch.float16)
    n, hits, history = 0, 0, []
    sel = np.zeros((NG, GROUP), dtype=np.uint8)
    line_of: List[int] = []
    for gi in range(NG):
        g = groups[gi]
        seen = gi + 1
        warm = n < warmup
        cached = (float("inf"), -1, None)
        if not warm:
            recent = history[-min(len(history), window):]
            cutoff = max((sum(recent) / len(recent)) * 0.99, acceptable)
            cached = min_mse(g, lines[:n])
            if cached[0] < cutoff:
                hits += 1
                line_of.append(cached[1])
                sel[gi] = cached[2].numpy()
                continue
        if n >= max_lines:
            line_of.append(cached[1])
            sel[gi] = cached[2].numpy()
            continue
        space = space_of(g, (hits / seen) > 0.6 or warm)
        new = min_mse(g, space)
        if new[0] >= cached[0]:
            line_of.append(cached[1])
            sel[gi] = cached[2].numpy()
            continue
        cand = space[new[1]]
        close = (lines - cand.unsqueeze(0)).abs().sum(-1) < cand.abs().sum(-1) * 0.0001
        if bool(close.any()):
            at = int(close.nonzero(as_tuple=True)[0][0])
        else:
            lines[n] = cand
            at = n
            n += 1
        line_of.append(at)
        sel[gi] = new[2].numpy()
        history.append(new[0])
    return {"sel": sel, "line_of": np.array(line_of), "lines": lines[:n].numpy().copy(), "hits": hits, "Kp": Kp}
