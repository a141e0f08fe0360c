"""The SBVR encoder on B200: dense fp16 tensor -> bit-planes + codebook (reference `_encode_to_sbvr`, sbvr/core.py:655-805).

The reference walks the groups of 256 values one by one in Python and, for each, materialises the squared differences
to every candidate coefficient line as tensors.  What it decides per group is kept here exactly:

  * after a warm-up of `cache_warmup_num` codebook lines, a group first looks for the best line already in the codebook
    and takes it if its MSE is below 0.99 x the mean MSE of the last `mse_window_size` accepted searches
    (sbvr/core.py:555-577);
  * otherwise (and while the codebook has room) it builds the group's own search space from the group's statistics
    (:400-483, :368-386), takes the best candidate, and if that beats the codebook's best, stores it as a new line
    (or reuses a line within 0.01 % of it) (:605-653).

How it is computed is different: the MSEs come from `sbvr_encode_mse_f16` (one thread per (group, candidate), nothing
of size candidates x 256 x 2^S is ever stored), and the codebook look-up runs for a whole batch of groups in one launch.
Because a group's decision depends on the codebook as its predecessors left it, the batch is speculative: the host
replays the decisions in order, and when a group adds a line, only that one line is evaluated against the rest of the
batch.  The result is the same as the sequential walk.

The search space of a group is generated with the same tensor operations and the same fp16 roundings as the
reference's; `space_device` says where ("cpu" reproduces a reference run on CPU bit for bit, "cuda" is what the
reference does when a GPU is present and is much faster).
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from . import _lib

GROUP = 256


@dataclass
class EncoderConfig:
    """The knobs of the reference's `_sbvr_enc_conf` (sbvr/core.py:19-37) that the data-difference error function uses."""
    num_sums: int = 4
    r_search_num: int = 64
    b_search_num: int = 40
    s_search_num: int = 40
    error_function: str = "data_diff_mse"
    mse_window_size: int = 20
    search_extend_ratio: float = 1.2
    cache_warmup_num: int = 10
    acceptable_mse: float = 10 ** -12
    extend_ratio: float = 1.2
    max_cache_lines: int = 2 ** 16
    batch_groups: int = 256            # groups looked up in the codebook per launch
    space_device: str = "cuda"
    mse_history: List[float] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> "EncoderConfig":
        d = dict(d or {})
        known = {k: d[k] for k in list(d) if k in cls.__dataclass_fields__}
        conf = cls(**known)
        if conf.error_function != "data_diff_mse":
            raise ValueError("only the data_diff_mse error function is implemented (the reference's other one is unfinished)")
        if not 1 <= conf.num_sums <= 4:
            raise ValueError("the GPU encoder covers num_sums 1..4")
        return conf


def _bin_combs(S: int, device, dtype=torch.float16) -> torch.Tensor:
    """[2^S, S] rows of 0/1, first column = most significant selector bit (sbvr/core.py:345-351)."""
    return torch.tensor(list(itertools.product([0, 1], repeat=S)), dtype=dtype, device=device)


# ---------------------------------------------------------------------------------------------------------------
# the candidate lines of one group
# ---------------------------------------------------------------------------------------------------------------
def _ratio_bias_scale_lines(r_list, b_list, s_list, S: int) -> torch.Tensor:
    """Lines b + s * (1, r, r^2, ..) / span(r) for every (b, s, r), b outermost, r innermost
    (`_get_coeff_search_space_from_lists`, sbvr/core.py:388-398); span = max - min over the 2^S sums of the powers."""
    powers = r_list.unsqueeze(1) ** torch.arange(S, device=r_list.device).unsqueeze(0)         # [R, S]
    sums = powers @ _bin_combs(S, r_list.device, r_list.dtype).T                               # [R, 2^S]
    unit = powers / (sums.max(dim=1)[0] - sums.min(dim=1)[0]).unsqueeze(1)
    scaled = s_list.view(-1, 1, 1) * unit.unsqueeze(0)                                         # [Sn, R, S]
    return (b_list.view(-1, 1, 1, 1) + scaled.unsqueeze(0)).view(-1, S)


def _grid_lines(data: torch.Tensor, conf: EncoderConfig, S: int, extended: bool) -> torch.Tensor:
    """A plain grid over the data range, one axis per coefficient (`_get_additional_search_space`, sbvr/core.py:368-386)."""
    budget = conf.r_search_num * conf.b_search_num * conf.s_search_num * 1.4
    if extended:
        budget *= conf.search_extend_ratio ** 3
    per_dim = int(budget ** (1 / S))
    lo, hi = torch.min(data), torch.max(data)
    edges = torch.linspace(lo, hi, S + 1, device=data.device, dtype=data.dtype)
    axes = []
    for i in range(S):
        slack = abs(edges[i]) * 0.8
        axes.append(torch.linspace(edges[i] - slack, edges[i + 1] + slack, per_dim + 1, device=data.device,
                                   dtype=data.dtype))
    return torch.cartesian_prod(*axes).view(-1, S)


def group_search_space(data: torch.Tensor, conf: EncoderConfig, extended: bool) -> torch.Tensor:
    """Candidate lines [n, S] (fp16, each sorted by magnitude) for one group of values `data` (fp16, on the device the
    space is to be generated on): `_get_coeff_search_space`, sbvr/core.py:400-483.  Every quantity has the type it has
    there (fp16 tensors for the data statistics, an fp32 tensor for the 95 % quantile, Python floats for the ratio
    ranges), because the fp16 roundings decide the candidates."""
    S = conf.num_sums
    d_max, d_avg, d_min = torch.max(data), torch.mean(data), torch.min(data)
    d_95 = torch.quantile(data.to(torch.float), 0.95)

    r_lo = (math.pi / 6, 0.94)                    # ratios below one ...
    r_hi = (1.06, math.pi * 2 / 3)                # ... and above
    r_lo_step = (r_lo[1] - r_lo[0]) / (conf.r_search_num / 2)
    r_hi_step = (r_hi[1] - r_hi[0]) / (conf.r_search_num / 2)
    b_hi = abs(d_avg) * 2.0 / S
    if b_hi < 0.3:
        b_hi = 0.3
    b_lo = -b_hi
    b_step = (b_hi - b_lo) / conf.b_search_num
    s_hi = (d_max - d_min) * 1.1
    s_lo = 2 * d_95
    s_step = (s_hi - s_lo) / conf.s_search_num
    if extended:
        r_lo_step /= conf.extend_ratio
        r_hi_step /= conf.extend_ratio
        b_step /= conf.extend_ratio
        s_step /= conf.extend_ratio

    kw = dict(device=data.device, dtype=data.dtype)
    r_list = torch.cat((-torch.arange(r_lo[0] + r_lo_step, r_lo[1] + r_lo_step, r_lo_step, **kw),
                        -torch.arange(r_hi[0] + r_hi_step, r_hi[1] + r_hi_step, r_hi_step, **kw)))
    s_list = torch.arange(s_lo + s_step, s_hi + s_step, s_step, **kw) if s_step != 0 else torch.tensor([s_lo], **kw)
    b_list = torch.arange(b_lo, b_hi, b_step, **kw) if b_step != 0 else torch.tensor([b_lo], **kw)

    space = _ratio_bias_scale_lines(r_list, b_list, s_list, S)
    if S <= 6:
        space = torch.cat((space, _grid_lines(data, conf, S, extended)), dim=0)
    order = torch.sort(space.abs(), dim=1)[1]
    return torch.gather(space, dim=1, index=order).contiguous()


# ---------------------------------------------------------------------------------------------------------------
# device helpers (thin wrappers of the C ABI)
# ---------------------------------------------------------------------------------------------------------------
def _mse(data: torch.Tensor, lines: torch.Tensor, S: int) -> torch.Tensor:
    """fp32 [groups, L]: MSE of every group of `data` [groups, 256] against every line of `lines` [L, S]."""
    groups, L = data.shape[0], lines.shape[0]
    out = torch.empty((groups, L), dtype=torch.float32, device=data.device)
    st = torch.cuda.current_stream(data.device).cuda_stream
    for g0 in range(0, groups, 32768):                      # grid.y limit
        g1 = min(groups, g0 + 32768)
        _lib.check(_lib.lib.sbvr_encode_mse_f16(data[g0:g1].data_ptr(), g1 - g0, lines.data_ptr(), L, S,
                                                out[g0:g1].data_ptr(), st), "sbvr_encode_mse_f16")
    return out


def _select(data: torch.Tensor, lines: torch.Tensor, which: torch.Tensor, S: int, sel_out: torch.Tensor) -> None:
    """sel_out[b] (uint8 [groups, 256]) = nearest-sum selectors of group b for line which[b] of `lines`."""
    st = torch.cuda.current_stream(data.device).cuda_stream
    _lib.check(_lib.lib.sbvr_encode_select_f16(data.data_ptr(), data.shape[0], lines.data_ptr(), which.data_ptr(), S,
                                               sel_out.data_ptr(), st), "sbvr_encode_select_f16")


def pack_selectors(sel: torch.Tensor, S: int) -> torch.Tensor:
    """Selectors uint8 [N, Kp] (device) -> bvr uint32 [Kp/32, N, S]."""
    N, Kp = sel.shape
    bvr = torch.empty((Kp // 32, N, S), dtype=torch.int32, device=sel.device)
    st = torch.cuda.current_stream(sel.device).cuda_stream
    _lib.check(_lib.lib.sbvr_encode_pack(sel.data_ptr(), N, Kp, S, bvr.data_ptr(), st), "sbvr_encode_pack")
    return bvr.view(torch.uint32)


# ---------------------------------------------------------------------------------------------------------------
# the walk over the groups
# ---------------------------------------------------------------------------------------------------------------
class _Codebook:
    """The growing coefficient cache and the running statistics that steer the search (the mutable part of the
    reference's `_sbvr_enc_conf`: coeff_cache, num_coeff_cache_lines, mse_history, cache_hits, group_idx)."""

    def __init__(self, conf: EncoderConfig, device):
        self.conf = conf
        self.lines = torch.zeros((conf.max_cache_lines, conf.num_sums), dtype=torch.float16, device=device)
        self.n = 0
        self.hits = 0
        self.seen = 0
        self.history: List[float] = list(conf.mse_history)

    def cutoff(self) -> float:
        """0.99 x the mean MSE of the most recent accepted searches, not below `acceptable_mse` (sbvr/core.py:563-568)."""
        window = self.history[-min(len(self.history), self.conf.mse_window_size):]
        return max((sum(window) / len(window)) * 0.99, self.conf.acceptable_mse)

    def find_or_add(self, line: torch.Tensor) -> Tuple[int, bool]:
        """Index of a stored line within 0.01 % (summed magnitude, fp16 arithmetic) of `line`, else the index it is
        appended at (sbvr/core.py:634-646).  Returns (index, appended)."""
        if self.n:
            diff = self.lines[:self.n] - line.unsqueeze(0)
            close = diff.abs().sum(-1) < line.abs().sum(-1) * 0.0001
            if bool(close.any()):
                return int(close.nonzero(as_tuple=True)[0][0]), False
        self.lines[self.n] = line
        self.n += 1
        return self.n - 1, True


def _full_search(group: torch.Tensor, book: _Codebook, extended: bool) -> Tuple[float, int, torch.Tensor]:
    """Best candidate of the group's own search space: (mse, index, the space [n, S] on the GPU)."""
    conf = book.conf
    src = group if conf.space_device == "cuda" else group.to(conf.space_device)
    space = group_search_space(src, conf, extended).to(group.device)
    mse = _mse(group.view(1, GROUP), space, conf.num_sums)[0]
    at = torch.argmin(mse)                                   # the first of equal minima, like the reference's argmin
    return float(mse[at]), int(at), space


@torch.inference_mode()
def encode(data: torch.Tensor, conf: EncoderConfig, device: Optional[torch.device] = None, progress=None):
    """Dense tensor [..., K] -> (bvr uint32 [Kp/32, N, S], coeff_idx uint8|uint16 [Kp/256, N], coeff_cache fp16 [C, S],
    stats) in the reference's GPU layout, N = product of the leading dimensions, Kp = K rounded up to 256 (zero padded,
    sbvr/core.py:667-676)."""
    dev = torch.device(device) if device is not None else torch.device("cuda")
    if dev.type != "cuda":
        raise RuntimeError("the encoder runs on a CUDA device (there is no CPU implementation)")
    S = conf.num_sums
    K = int(data.shape[-1])
    Kp = (K + GROUP - 1) // GROUP * GROUP
    flat = data.reshape(-1, K).to(dev).to(torch.float16)
    N = flat.shape[0]
    if Kp != K:
        flat = torch.nn.functional.pad(flat, (0, Kp - K))
    groups = flat.contiguous().view(-1, GROUP)               # group i = (row i // (Kp/256), block i % (Kp/256))
    NG = groups.shape[0]
    with torch.cuda.device(dev):
        book = _Codebook(conf, dev)
        sel = torch.empty((NG, GROUP), dtype=torch.uint8, device=dev)
        line_of = [0] * NG
        one = torch.zeros(1, dtype=torch.int32, device=dev)

        def select_from(space: torch.Tensor, at: int, gi: int):
            one.fill_(at)
            _select(groups[gi:gi + 1], space, one, S, sel[gi:gi + 1])

        def search_and_store(gi: int, cached_mse: float, cached_at: int, warm: bool) -> Tuple[bool, Optional[int]]:
            """The miss path of one group.  Returns (the stored line `cached_at` was kept, index of an appended line)."""
            hitrate = book.hits / book.seen
            new_mse, at, space = _full_search(groups[gi], book, hitrate > 0.6 or warm)
            if new_mse >= cached_mse:                        # the codebook already has something at least as good
                line_of[gi] = cached_at
                return True, None
            idx, appended = book.find_or_add(space[at])
            line_of[gi] = idx
            select_from(space, at, gi)                       # selectors of the candidate itself, also when an old line is reused
            book.history.append(new_mse)
            return False, (idx if appended else None)

        gi = 0
        while gi < NG:
            if book.n < conf.cache_warmup_num:               # warm-up: every group searches its own space
                book.seen += 1
                search_and_store(gi, float("inf"), -1, True)
                gi += 1
                if progress:
                    progress(gi, NG)
                continue
            g1 = min(NG, gi + conf.batch_groups)
            mse = _mse(groups[gi:g1], book.lines[:book.n], S)
            at = torch.argmin(mse, dim=1)
            best_mse = mse.gather(1, at.unsqueeze(1)).squeeze(1).tolist()
            best_at = at.tolist()
            from_book = []                                   # groups of this batch whose selectors come from a stored line
            for b in range(g1 - gi):
                g = gi + b
                book.seen += 1
                if best_mse[b] < book.cutoff():
                    book.hits += 1
                    line_of[g] = best_at[b]
                    from_book.append(g)
                    continue
                if book.n >= conf.max_cache_lines:           # full codebook: the best stored line has to do
                    line_of[g] = best_at[b]
                    from_book.append(g)
                    continue
                kept, added = search_and_store(g, best_mse[b], best_at[b], False)
                if kept:
                    from_book.append(g)
                if added is not None and g + 1 < g1:         # the rest of the batch has not seen the new line yet
                    extra = _mse(groups[g + 1:g1], book.lines[added:added + 1], S)[:, 0].tolist()
                    for r, m in enumerate(extra):
                        if m < best_mse[b + 1 + r]:
                            best_mse[b + 1 + r], best_at[b + 1 + r] = m, added
            if from_book:
                rows = torch.tensor(from_book, dtype=torch.long, device=dev)
                which = torch.tensor([line_of[g] for g in from_book], dtype=torch.int32, device=dev)
                tmp = torch.empty((len(from_book), GROUP), dtype=torch.uint8, device=dev)
                _select(groups[rows].contiguous(), book.lines, which, S, tmp)
                sel[rows] = tmp
            gi = g1
            if progress:
                progress(gi, NG)

        C = book.n
        cache = book.lines[:C].contiguous()
        idx = torch.tensor(line_of, dtype=torch.int32, device=dev).view(N, Kp // GROUP).T.contiguous()
        idx = idx.to(torch.uint8) if C <= 256 else idx.to(torch.int16).view(torch.uint16)   # C <= 65536: the bits fit
        bvr = pack_selectors(sel.view(N, Kp), S)
        torch.cuda.synchronize(dev)
    stats = {"groups": NG, "cache_lines": C, "cache_hits": book.hits, "searches": len(book.history) - len(conf.mse_history)}
    return bvr, idx, cache, stats
