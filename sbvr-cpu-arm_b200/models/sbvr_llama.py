"""Llama decoder built on SBVR linears: `SBVRLinear`, `SBVRLlamaForCausalLM` (prefill, greedy decode under a CUDA
graph, tensor parallel over NCCL).

The reference model (models/sbvr_llama.py) is a re-vendored HuggingFace Llama whose `SBVRLinear` (:66-106) is a
stub: its weights are decoded to dense fp16 before use (sbvr_utils/utils_llama.py:132-158) and every layer runs
about fifteen eager launches.  Here every projection stays packed and runs through `sbvr.linear`; q/k/v and
gate/up are fused into one linear each (the packed layout concatenates along N); the ops between the linears
are the library's fused kernels.  Arithmetic follows the reference's modules:
  LlamaRMSNorm.forward :118-123, LlamaRotaryEmbedding.forward / apply_rotary_pos_emb :169-224,
  LlamaMLP.forward :238-240, repeat_kv / eager_attention_forward :243-278, LlamaAttention.forward :307-354,
  LlamaDecoderLayer.forward :368-408, LlamaModel.forward :568-672, SBVRLlamaForCausalLM.forward :836-924.

Tensor parallel (one process per GPU): q/k/v, gate/up and lm_head are split over output rows, o and down over
input columns; the two row-parallel outputs of a layer are summed with an all-reduce (torch.distributed, NCCL),
which is captured into the decode graph together with the kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

import sbvr as _sbvr
from sbvr import _lib
from sbvr.core import XOP_ADD_RMSNORM, XOP_DIGITS, XOP_NONE, XOP_SILU_MUL, linear_fused
from sbvr.core import linear as sbvr_linear
from sbvr.core import sbvr as sbvr_tensor

from . import parallel


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_position_embeddings: int = 8192
    # SBVR encoding of every linear
    num_sums: int = 4
    group_len: int = 256
    codebook_lines: int = 4096

    @staticmethod
    def preset(name: str) -> "LlamaConfig":
        if name in ("llama3-8b", "8b"):
            return LlamaConfig()
        if name in ("llama3-70b", "70b"):
            return LlamaConfig(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                               num_attention_heads=64, num_key_value_heads=8)
        if name == "tiny":
            return LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                               num_key_value_heads=2, vocab_size=1024, codebook_lines=256,
                               max_position_embeddings=512)
        if name == "tiny8":                        # splits over up to eight tensor-parallel ranks: eight KV heads, and
            # eight 256-column groups in the inputs of the row-parallel projections (o: hidden, down: intermediate)
            return LlamaConfig(hidden_size=2048, intermediate_size=4096, num_hidden_layers=2, num_attention_heads=16,
                               num_key_value_heads=8, vocab_size=1024, codebook_lines=256,
                               max_position_embeddings=512)
        raise ValueError(f"unknown preset {name}")

    def tp_problems(self, world: int, group_len: int = 256) -> list:
        """Why this configuration cannot be split over `world` tensor-parallel ranks (empty list: it can)."""
        bad = []
        if self.num_attention_heads % world:
            bad.append(f"{self.num_attention_heads} attention heads over {world} ranks")
        if self.num_key_value_heads % world:
            bad.append(f"{self.num_key_value_heads} KV heads over {world} ranks")
        for name, k in (("hidden_size", self.hidden_size), ("intermediate_size", self.intermediate_size)):
            if k % (world * group_len):
                bad.append(f"{name} {k}: the row-parallel projection's input does not split into {world} x groups of {group_len}")
        if self.vocab_size % world:
            bad.append(f"vocabulary {self.vocab_size} over {world} ranks")
        return bad


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class SBVRLinear(torch.nn.Module):
    """`y = x @ W.T (+ bias)` with W held as a packed `sbvr` tensor.  Takes the place of the reference's stub of
    the same name (models/sbvr_llama.py:66-106), whose forward multiplied by a weight restored to dense fp16."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, num_sums: int = 4,
                 group_len: int = 256):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.num_sums = num_sums
        self.group_len = group_len
        self.weight: Optional[sbvr_tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self._has_bias = bias

    @classmethod
    def from_sbvr(cls, w: sbvr_tensor, bias: Optional[torch.Tensor] = None) -> "SBVRLinear":
        m = cls(int(w.original_data_shape[-1]), w.out_features, bias is not None, w.num_sums, w.bvr_len)
        m.weight = w
        m.bias = bias
        return m

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.weight is None:
            raise RuntimeError("SBVRLinear has no weight: build it with from_sbvr or load a packed file")
        return sbvr_linear(x, self.weight, self.bias, out=out)

    def packed_bytes(self) -> int:
        w = self.weight
        n = w.bvr.numel() * 4 + w.coeff_cache.numel() * 2
        if w.coeff_idx is not None:
            n += w.coeff_idx.numel() * w.coeff_idx.element_size()
        return n


def synthetic_packed(N: int, K: int, S: int, G: int, C: int, gen: torch.Generator, device) -> dict:
    """Random packed weight in the reference's layout: Bernoulli(1/2) plane bits, codebook lines ~ N(0, 0.01^2)
    sorted by magnitude, uniform indices.  Stands in for an encoded checkpoint (none can be downloaded here)."""
    bvr = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 32, N, S), dtype=torch.int32, device=device, generator=gen)
    cache = torch.randn((C, S), device=device, generator=gen) * 0.01
    order = cache.abs().argsort(dim=1, descending=True)
    cache = torch.gather(cache, 1, order).half()
    idx = torch.randint(0, C, (K // G, N), device=device, generator=gen, dtype=torch.int32)
    idx = idx.to(torch.uint8) if C <= 256 else idx.to(torch.int16).view(torch.uint16)
    return {"bvr": bvr, "coeff_idx": idx, "coeff_cache": cache}


def _make_linear(packed: dict, G: int, device) -> SBVRLinear:
    w = sbvr_tensor.from_packed(packed["bvr"], packed["coeff_idx"], packed["coeff_cache"], group_len=G,
                                device=torch.device(device))
    return SBVRLinear.from_sbvr(w)


class SBVRLlamaDecoderLayer(torch.nn.Module):
    def __init__(self, qkv: SBVRLinear, o: SBVRLinear, gate_up: SBVRLinear, down: SBVRLinear,
                 input_norm: torch.Tensor, post_norm: torch.Tensor):
        super().__init__()
        self.qkv_proj, self.o_proj, self.gate_up_proj, self.down_proj = qkv, o, gate_up, down
        self.input_layernorm_weight = input_norm
        self.post_attention_layernorm_weight = post_norm


@dataclass
class _Buffers:
    """Activations of one forward of `tokens` rows; allocated once so that a captured graph stays valid."""
    tokens: int
    ids: torch.Tensor
    positions: torch.Tensor
    h: torch.Tensor
    h2: torch.Tensor
    xn: torch.Tensor
    qkv: torch.Tensor
    ao: torch.Tensor
    o: torch.Tensor
    gu: torch.Tensor
    act: torch.Tensor
    down: torch.Tensor
    logits: torch.Tensor
    next_ids: torch.Tensor
    att_scratch: Optional[torch.Tensor]
    all_logits: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)


class SBVRLlamaForCausalLM(torch.nn.Module):
    """Greedy-decoding Llama on packed weights.  `tp_group` = a torch.distributed process group whose ranks hold
    one shard each (None = single GPU)."""

    def __init__(self, config: LlamaConfig, device="cuda", tp_group=None, max_batch: int = 1, max_ctx: int = 2048):
        super().__init__()
        self.config = config
        self.device = torch.device(device)
        self.tp_group = tp_group
        self.tp_size = 1 if tp_group is None else torch.distributed.get_world_size(tp_group)
        problems = config.tp_problems(self.tp_size, config.group_len if hasattr(config, "group_len") else 256)
        if problems:
            raise ValueError("configuration does not split over the tensor-parallel ranks: " + "; ".join(problems))
        self.tp_rank = 0 if tp_group is None else torch.distributed.get_rank(tp_group)
        c = config
        if c.head_dim != 128:
            raise ValueError("the attention kernel serves head_dim 128")
        if c.num_attention_heads % self.tp_size or c.num_key_value_heads % self.tp_size:
            raise ValueError("heads must divide over the tensor-parallel ranks")
        self.n_heads = c.num_attention_heads // self.tp_size
        self.n_kv = c.num_key_value_heads // self.tp_size
        self.inter = c.intermediate_size // self.tp_size
        self.vocab_local = c.vocab_size // self.tp_size
        self.max_batch, self.max_ctx = max_batch, max_ctx
        self.layers: List[SBVRLlamaDecoderLayer] = []
        self.embed_tokens: Optional[torch.Tensor] = None
        self.norm_weight: Optional[torch.Tensor] = None
        self.lm_head: Optional[SBVRLinear] = None
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))
        self.inv_freq = inv.to(self.device)
        self.attention_scaling = 1.0
        self.kcache: List[torch.Tensor] = []
        self.vcache: List[torch.Tensor] = []
        self._bufs = {}
        self._graph = None
        self._stream = None
        self._comm = None
        self.fuse_glue = True                      # fold norm / SiLU into the decode linears where the kernel allows
        self.pushed_allreduce = True               # tensor-parallel decode: results pushed to the peers by the GEMV itself
        self._argmax_scratch = torch.empty(256, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ weights
    @torch.inference_mode()
    def init_synthetic(self, seed: int = 7) -> "SBVRLlamaForCausalLM":
        """Random-init weights of the configured architecture (every rank draws the full tensors from the same
        seed and keeps its shard, so a tensor-parallel model equals the single-GPU one)."""
        c, dev = self.config, self.device
        S, G, C = c.num_sums, c.group_len, c.codebook_lines
        gen = torch.Generator(device=dev).manual_seed(seed)
        H, I = c.hidden_size, c.intermediate_size
        qd, kvd = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        r, n = self.tp_rank, self.tp_size
        self.embed_tokens = (torch.randn((c.vocab_size, H), device=dev, generator=gen) * 0.02).half()
        for _ in range(c.num_hidden_layers):
            q = synthetic_packed(qd, H, S, G, C, gen, dev)
            k = synthetic_packed(kvd, H, S, G, C, gen, dev)
            v = synthetic_packed(kvd, H, S, G, C, gen, dev)
            o = synthetic_packed(H, qd, S, G, C, gen, dev)
            gate = synthetic_packed(I, H, S, G, C, gen, dev)
            up = synthetic_packed(I, H, S, G, C, gen, dev)
            down = synthetic_packed(H, I, S, G, C, gen, dev)
            # projections that are fused into one linear share a codebook in the synthetic model, so that the
            # fused codebook stays small enough for the kernels to keep it in shared memory
            k["coeff_cache"] = v["coeff_cache"] = q["coeff_cache"]
            up["coeff_cache"] = gate["coeff_cache"]
            qkv = parallel.fuse_rows([parallel.shard_rows(q, r, n), parallel.shard_rows(k, r, n),
                                      parallel.shard_rows(v, r, n)])
            gu = parallel.fuse_rows([parallel.shard_rows(gate, r, n), parallel.shard_rows(up, r, n)])
            layer = SBVRLlamaDecoderLayer(_make_linear(qkv, G, dev), _make_linear(parallel.shard_cols(o, r, n, G), G, dev),
                                          _make_linear(gu, G, dev), _make_linear(parallel.shard_cols(down, r, n, G), G, dev),
                                          torch.ones(H, dtype=torch.float16, device=dev),
                                          torch.ones(H, dtype=torch.float16, device=dev))
            self.layers.append(layer)
            del q, k, v, o, gate, up, down, qkv, gu
        self.norm_weight = torch.ones(H, dtype=torch.float16, device=dev)
        head = synthetic_packed(c.vocab_size, H, S, G, C, gen, dev)
        self.lm_head = _make_linear(parallel.shard_rows(head, r, n), G, dev)
        self._alloc_cache()
        return self

    def enable_fused_allreduce(self, max_rows: int = 16) -> bool:
        """Tensor parallel only: route the all-reduces of up to `max_rows` activation rows through the fused
        peer-memory kernel.  Returns False (and keeps NCCL) when symmetric memory cannot be set up here."""
        if self.tp_size == 1 and self.tp_group is None:
            return False
        from .comm import SymmetricAllReduce
        try:
            self._comm = SymmetricAllReduce(self.tp_group, self.device, max_rows, self.config.hidden_size,
                                            2 * self.config.num_hidden_layers)
        except Exception as e:                     # no peer mapping on this machine: NCCL stays
            self._comm_error = repr(e)
            self._comm = None
        self._graph = None
        return self._comm is not None

    def set_pushed_allreduce(self, on: bool) -> None:
        """Decode (up to four rows): whether the row-parallel linears push their results into the ranks' receive areas
        (on by default) or write partials that the one-shot all-reduce kernel then reads over NVLink."""
        self.pushed_allreduce = bool(on)
        self._graph = None

    def _alloc_cache(self):
        c = self.config
        shape = (self.max_batch, self.n_kv, self.max_ctx, c.head_dim)
        self.kcache = [torch.zeros(shape, dtype=torch.float16, device=self.device) for _ in range(c.num_hidden_layers)]
        self.vcache = [torch.zeros(shape, dtype=torch.float16, device=self.device) for _ in range(c.num_hidden_layers)]

    def packed_weight_bytes(self) -> int:
        n = sum(l.qkv_proj.packed_bytes() + l.o_proj.packed_bytes() + l.gate_up_proj.packed_bytes() +
                l.down_proj.packed_bytes() for l in self.layers)
        return n + self.lm_head.packed_bytes()

    # ------------------------------------------------------------------ buffers
    def _act(self, tokens: int, rows_out: int) -> _Buffers:
        key = (tokens, rows_out)
        b = self._bufs.get(key)
        if b is not None:
            return b
        c, dev = self.config, self.device
        f16 = dict(dtype=torch.float16, device=dev)
        H = c.hidden_size
        nsplit = self._nsplit(tokens)
        b = _Buffers(
            tokens=tokens,
            ids=torch.zeros(tokens, dtype=torch.int32, device=dev),
            positions=torch.zeros(tokens, dtype=torch.int32, device=dev),
            h=torch.empty((tokens, H), **f16), h2=torch.empty((tokens, H), **f16), xn=torch.empty((tokens, H), **f16),
            qkv=torch.empty((tokens, (self.n_heads + 2 * self.n_kv) * c.head_dim), **f16),
            ao=torch.empty((tokens, self.n_heads * c.head_dim), **f16), o=torch.empty((tokens, H), **f16),
            gu=torch.empty((tokens, 2 * self.inter), **f16), act=torch.empty((tokens, self.inter), **f16),
            down=torch.empty((tokens, H), **f16),
            logits=torch.empty((rows_out, self.vocab_local), **f16),
            next_ids=torch.zeros(rows_out, dtype=torch.int32, device=dev),
            att_scratch=(torch.zeros(tokens * self.n_heads * nsplit * 130 + tokens * self.n_kv, dtype=torch.float32,
                                     device=dev) if nsplit > 1 else None))
        if self.tp_size > 1:
            b.extra["gathered"] = torch.empty((self.tp_size, rows_out, self.vocab_local), **f16)
        self._bufs[key] = b
        return b

    def _nsplit(self, tokens: int) -> int:
        # decode with few tokens: split the context so that about one CTA per SM works
        ctas = tokens * self.n_kv
        return 1 if ctas >= 96 else max(1, min(16, 192 // ctas))

    # ------------------------------------------------------------------ one forward over `tokens` rows
    def _all_reduce(self, t: torch.Tensor):
        if self.tp_size > 1:
            torch.distributed.all_reduce(t, group=self.tp_group)

    def _forward_rows(self, b: _Buffers, tokens_per_seq: int, last_only: bool):
        """Runs embedding -> layers -> norm -> lm_head on the rows described by b.ids / b.positions.
        `last_only`: logits (and argmax) only for the last token of every sequence."""
        c, L = self.config, _lib.lib
        st = _stream()
        T, H = b.tokens, c.hidden_size
        eps = float(c.rms_norm_eps)
        scale = 1.0 / math.sqrt(c.head_dim)
        nsplit = self._nsplit(T)
        ck = _lib.check
        # Tensor parallel with few rows: the partial outputs of o and down go to symmetric memory and one fused
        # kernel all-reduces them, adds the residual and applies the next RMSNorm.  Otherwise NCCL + add_rmsnorm.
        comm = self._comm if (self._comm is not None and T <= self._comm.max_rows) else None
        ws = _lib.workspace(self.device.index or 0, st) if comm is not None else None
        n_layers = len(self.layers)
        # Up to four rows (decode): the residual add + RMSNorm in front of q|k|v, gate|up and lm_head and the
        # SiLU * up in front of down are folded into those linears' kernels.  The folded norm cannot update the
        # residual in place (other CTAs still read it), so the residual alternates between two buffers.
        fuse = self.fuse_glue and T <= 4
        hc, ho = b.h, b.h2                         # current residual, spare buffer

        def norm_linear(lin, delta, weight, out, keep_residual=True):
            """out = lin(rmsnorm(hc + delta) * weight); the residual becomes hc + delta."""
            nonlocal hc, ho
            if fuse and isinstance(lin, SBVRLinear) and linear_fused(
                    XOP_ADD_RMSNORM, hc, lin.weight, out, delta=delta, norm_weight=weight,
                    h_out=ho if keep_residual else None, eps=eps, bias=lin.bias):
                if keep_residual:
                    hc, ho = ho, hc
                return
            ck(L.sbvr_add_rmsnorm_f16(hc.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                      hc.data_ptr() if keep_residual else None, b.xn.data_ptr(), T, H, eps, st), "rmsnorm")
            lin(b.xn, out=out)

        ck(L.sbvr_embedding_f16(b.ids.data_ptr(), self.embed_tokens.data_ptr(), hc.data_ptr(), T, H, st), "embedding")
        delta, normed, digits = None, False, False
        for li, layer in enumerate(self.layers):
            if normed:
                if not (digits and linear_fused(XOP_DIGITS, b.xn, layer.qkv_proj.weight, b.qkv, bias=layer.qkv_proj.bias)):
                    layer.qkv_proj(b.xn, out=b.qkv)
                digits = False
            else:
                norm_linear(layer.qkv_proj, delta, layer.input_layernorm_weight, b.qkv)
            att_scratch = None if b.att_scratch is None else b.att_scratch.data_ptr()
            if tokens_per_seq == 1 and self.fuse_glue:     # decode: rotary embedding and cache append inside attention
                ck(L.sbvr_rope_attention_f16(b.qkv.data_ptr(), b.positions.data_ptr(), self.inv_freq.data_ptr(),
                                             float(self.attention_scaling), self.kcache[li].data_ptr(),
                                             self.vcache[li].data_ptr(), b.ao.data_ptr(), att_scratch, T, self.n_heads,
                                             self.n_kv, c.head_dim, self.max_ctx, scale, nsplit, st), "rope_attention")
            else:
                ck(L.sbvr_rope_append_f16(b.qkv.data_ptr(), b.positions.data_ptr(), self.inv_freq.data_ptr(),
                                          float(self.attention_scaling), self.kcache[li].data_ptr(),
                                          self.vcache[li].data_ptr(), T, tokens_per_seq, self.n_heads, self.n_kv,
                                          c.head_dim, self.max_ctx, st), "rope")
                ck(L.sbvr_attention_f16(b.qkv.data_ptr(), self.kcache[li].data_ptr(), self.vcache[li].data_ptr(),
                                        b.positions.data_ptr(), b.ao.data_ptr(), att_scratch, T, tokens_per_seq,
                                        self.n_heads, self.n_kv, c.head_dim, self.max_ctx, scale, nsplit, st), "attention")
            if comm is not None:
                # decode: the o projection pushes its result into every rank's receive area (no separate all-reduce)
                # rows longer than 4096: the reduce kernel also leaves the normalised rows as the digits of the next GEMV
                want = fuse and comm.emits_digits(T) and isinstance(layer.gate_up_proj, SBVRLinear)
                if fuse and self.pushed_allreduce and isinstance(layer.o_proj, SBVRLinear) and comm.push_linear(
                        2 * li, XOP_NONE, b.ao, layer.o_proj.weight, T, bias=layer.o_proj.bias):
                    have = comm.ll_reduce_add_rmsnorm(2 * li, hc, layer.post_attention_layernorm_weight, b.xn, T, eps, ws,
                                                      st, emit_digits=want)
                else:
                    layer.o_proj(b.ao, out=comm.partial_out(2 * li, T))
                    have = comm.reduce_add_rmsnorm(2 * li, hc, layer.post_attention_layernorm_weight, b.xn, T, eps, ws, st,
                                                   emit_digits=want)
                if not (have and linear_fused(XOP_DIGITS, b.xn, layer.gate_up_proj.weight, b.gu,
                                              bias=layer.gate_up_proj.bias)):
                    layer.gate_up_proj(b.xn, out=b.gu)
            else:
                layer.o_proj(b.ao, out=b.o)
                self._all_reduce(b.o)
                norm_linear(layer.gate_up_proj, b.o, layer.post_attention_layernorm_weight, b.gu)
            down_out = comm.partial_out(2 * li + 1, T) if comm is not None else b.down
            pushed = (comm is not None and fuse and self.pushed_allreduce and isinstance(layer.down_proj, SBVRLinear) and
                      comm.push_linear(2 * li + 1, XOP_SILU_MUL, b.gu, layer.down_proj.weight, T, bias=layer.down_proj.bias))
            if not pushed and not (fuse and isinstance(layer.down_proj, SBVRLinear) and
                                   linear_fused(XOP_SILU_MUL, b.gu, layer.down_proj.weight, down_out, bias=layer.down_proj.bias)):
                ck(L.sbvr_silu_mul_f16(b.gu.data_ptr(), b.act.data_ptr(), T, self.inter, st), "silu_mul")
                layer.down_proj(b.act, out=down_out)
            if comm is not None:
                nw = self.layers[li + 1].input_layernorm_weight if li + 1 < n_layers else self.norm_weight
                nxt = self.layers[li + 1].qkv_proj if li + 1 < n_layers else None      # (lm_head rows may be selected first)
                want = fuse and comm.emits_digits(T) and isinstance(nxt, SBVRLinear)
                if pushed:
                    digits = comm.ll_reduce_add_rmsnorm(2 * li + 1, hc, nw, b.xn, T, eps, ws, st, emit_digits=want)
                else:
                    digits = comm.reduce_add_rmsnorm(2 * li + 1, hc, nw, b.xn, T, eps, ws, st, emit_digits=want)
                delta, normed = None, True
            else:
                self._all_reduce(b.down)
                delta, normed = b.down, False
        rows_sel = last_only and tokens_per_seq > 1
        if normed or rows_sel:
            if not normed:
                ck(L.sbvr_add_rmsnorm_f16(hc.data_ptr(), None if delta is None else delta.data_ptr(),
                                          self.norm_weight.data_ptr(), None, b.xn.data_ptr(), T, H, eps, st), "rmsnorm")
            rows = b.xn.view(-1, tokens_per_seq, H)[:, -1, :].contiguous() if rows_sel else b.xn
            self.lm_head(rows, out=b.logits)
        else:
            norm_linear(self.lm_head, delta, self.norm_weight, b.logits, keep_residual=False)
        if self._comm is not None:
            self._comm.end_step()
        if self.tp_size > 1:
            g = b.extra["gathered"]
            torch.distributed.all_gather_into_tensor(g, b.logits, group=self.tp_group)
            full = g.permute(1, 0, 2).reshape(b.logits.shape[0], -1).contiguous()
        else:
            full = b.logits
        ck(L.sbvr_argmax_f16(full.data_ptr(), b.next_ids.data_ptr(), self._argmax_scratch.data_ptr(), full.shape[0],
                             full.shape[1], st), "argmax")
        return full

    # ------------------------------------------------------------------ public API
    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Logits [B, L, vocab] of a prompt batch starting at position 0 (fills the KV cache)."""
        B, Lq = input_ids.shape
        if B > self.max_batch or Lq > self.max_ctx:
            raise ValueError("batch or length beyond the cache this model was built with")
        b = self._act(B * Lq, B * Lq)
        b.ids.copy_(input_ids.reshape(-1).to(torch.int32))
        b.positions.copy_(torch.arange(Lq, dtype=torch.int32, device=self.device).repeat(B))
        full = self._forward_rows(b, Lq, last_only=False)
        self._check()
        return full.view(B, Lq, -1)

    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Runs the prompt, fills the KV cache, returns the greedy next token of every sequence [B] (int32)."""
        B, Lq = input_ids.shape
        if B > self.max_batch or Lq > self.max_ctx:
            raise ValueError("batch or length beyond the cache this model was built with")
        b = self._act(B * Lq, B)
        b.ids.copy_(input_ids.reshape(-1).to(torch.int32))
        b.positions.copy_(torch.arange(Lq, dtype=torch.int32, device=self.device).repeat(B))
        self._forward_rows(b, Lq, last_only=True)
        return b.next_ids[:B].clone()

    @torch.inference_mode()
    def decode_step(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One eager decode step: `tokens` [B] at `positions` [B] -> greedy next tokens [B]."""
        B = tokens.shape[0]
        b = self._act(B, B)
        b.ids.copy_(tokens.to(torch.int32))
        b.positions.copy_(positions.to(torch.int32))
        self._forward_rows(b, 1, last_only=True)
        return b.next_ids[:B].clone()

    def _capture_decode(self, B: int):
        """Captures one decode step (all kernels, the all-reduces, the position increment) into a CUDA graph."""
        b = self._act(B, B)
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):                     # warm-up outside capture: workspaces, kernel attributes, NCCL
                self._forward_rows(b, 1, last_only=True)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            # thread_local: other threads (the NCCL watchdog) may touch the CUDA API while this one captures
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                self._forward_rows(b, 1, last_only=True)
                b.ids.copy_(b.next_ids)
                b.positions.add_(1)
        torch.cuda.current_stream().wait_stream(s)
        self._graph, self._stream, self._graph_B = g, s, B
        return g

    @torch.inference_mode()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, use_graph: bool = True) -> torch.Tensor:
        """Greedy generation: prefill, then `max_new_tokens - 1` decode steps.  Returns [B, max_new_tokens] int32."""
        B, Lq = input_ids.shape
        if Lq + max_new_tokens > self.max_ctx:
            raise ValueError("prompt + new tokens beyond the KV cache")
        out = torch.empty((B, max_new_tokens), dtype=torch.int32, device=self.device)
        nxt = self.prefill(input_ids)
        out[:, 0] = nxt
        b = self._act(B, B)
        b.ids.copy_(nxt)
        b.positions.fill_(Lq)
        if use_graph and (self._graph is None or self._graph_B != B):
            # the warm-up steps of the capture write cache slot Lq with the values the first real step writes again
            self._capture_decode(B)
        torch.cuda.synchronize(self.device)
        for i in range(1, max_new_tokens):
            if use_graph:
                self._graph.replay()
            else:
                self._forward_rows(b, 1, last_only=True)
                b.ids.copy_(b.next_ids)
                b.positions.add_(1)
            out[:, i] = b.next_ids
        self._check()
        return out

    def _check(self):
        torch.cuda.synchronize(self.device)
        for (dev, st), ws in list(_lib._workspaces.items()):
            rc = ws.status(st)
            if rc != 0:
                raise RuntimeError("sbvr: " + _lib.strerror(rc) + f" (wait 0x{_lib.lib.sbvr_last_timeout_where():x}, info {_lib.lib.sbvr_last_timeout_info(0)} 0x{_lib.lib.sbvr_last_timeout_info(1):x})")
