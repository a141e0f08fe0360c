"""TEST INFRASTRUCTURE - plain PyTorch restatement of the reference's Llama forward on dense weights.

Only tests may import this file; the product never does.

Follows the reference model op by op, in the dtypes the reference uses (fp16 tensors, fp32 islands):
  LlamaRMSNorm.forward                         models/sbvr_llama.py:118-123
  LlamaRotaryEmbedding.forward                 models/sbvr_llama.py:169-190
  rotate_half / apply_rotary_pos_emb           models/sbvr_llama.py:193-224
  LlamaMLP.forward                             models/sbvr_llama.py:238-240
  repeat_kv / eager_attention_forward          models/sbvr_llama.py:243-278
  LlamaAttention.forward                       models/sbvr_llama.py:307-354
  LlamaDecoderLayer.forward                    models/sbvr_llama.py:368-408
  LlamaModel.forward / SBVRLlamaForCausalLM    models/sbvr_llama.py:568-672, :836-924
with every linear computed as `x @ W.T` on the decoded weight, which is what the reference's flow does after
`sbvr_decompress_on_llama` (sbvr_utils/utils_llama.py:132-158).  Parity: unpinned by the reference (it holds no
whole-model test or fixture); this restatement is the pin.
"""
import math

import torch


def rmsnorm(x, weight, eps):
    dt = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return weight * xf.to(dt)


def rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope_cos_sin(positions, head_dim, theta, dtype, attention_scaling=1.0):
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    freqs = positions.to(torch.float32)[..., None] * inv_freq            # [B, L, d/2]
    emb = torch.cat((freqs, freqs), dim=-1)
    return (emb.cos() * attention_scaling).to(dtype), (emb.sin() * attention_scaling).to(dtype)


def repeat_kv(x, n_rep):
    b, h, l, d = x.shape
    if n_rep == 1:
        return x
    return x[:, :, None, :, :].expand(b, h, n_rep, l, d).reshape(b, h * n_rep, l, d)


def forward(params: dict, input_ids: torch.Tensor) -> torch.Tensor:
    """params: embed [V,H], layers = list of dicts (q,k,v,o,gate,up,down dense fp16 [N,K]; input_norm, post_norm [H]),
    norm [H], lm_head [V,H], n_heads, n_kv, head_dim, eps, theta.  Returns logits [B, L, V] (fp16)."""
    B, L = input_ids.shape
    nh, nkv, d = params["n_heads"], params["n_kv"], params["head_dim"]
    eps, theta = params["eps"], params["theta"]
    h = params["embed"][input_ids.long()]
    pos = torch.arange(L, device=h.device)[None, :].expand(B, L)
    cos, sin = rope_cos_sin(pos, d, theta, h.dtype)
    cos, sin = cos[:, None], sin[:, None]                                 # unsqueeze_dim = 1
    mask = torch.full((L, L), torch.finfo(h.dtype).min, dtype=h.dtype, device=h.device).triu(1)[None, None]
    scaling = d ** -0.5
    for lw in params["layers"]:
        residual = h
        x = rmsnorm(h, lw["input_norm"], eps)
        q = (x @ lw["q"].T).view(B, L, nh, d).transpose(1, 2)
        k = (x @ lw["k"].T).view(B, L, nkv, d).transpose(1, 2)
        v = (x @ lw["v"].T).view(B, L, nkv, d).transpose(1, 2)
        q = (q * cos) + (rotate_half(q) * sin)
        k = (k * cos) + (rotate_half(k) * sin)
        kk, vv = repeat_kv(k, nh // nkv), repeat_kv(v, nh // nkv)
        w = torch.matmul(q, kk.transpose(2, 3)) * scaling
        w = w + mask
        w = torch.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
        a = torch.matmul(w, vv).transpose(1, 2).contiguous().reshape(B, L, nh * d)
        h = residual + a @ lw["o"].T
        residual = h
        x = rmsnorm(h, lw["post_norm"], eps)
        m = (torch.nn.functional.silu(x @ lw["gate"].T) * (x @ lw["up"].T)) @ lw["down"].T
        h = residual + m
    h = rmsnorm(h, params["norm"], eps)
    return h @ params["lm_head"].T
