"""Pins the model oracle (`oracle/llama_ref.py`, the plain-PyTorch restatement of the reference's Llama forward,
reference models/sbvr_llama.py:109-408) to an independent implementation: the installed `transformers`
`LlamaForCausalLM` with eager attention, on the same random fp16 weights.  The reference vendors that very model file
(an older transformers release that cannot be imported here), so agreement with the installed one is the closest
available pin of whole-model semantics: RMSNorm, rotary embedding (theta, half rotation), grouped-query attention with
the causal mask, SwiGLU MLP, residual order, final norm and head.

Tolerance: max|logits - ref| / max|ref| <= 1e-2 (fp16 model; the two implementations round in slightly different places).
"""
import pytest
import torch

from oracle import llama_ref

TOL = 1e-2


def _hf_model(hidden, inter, layers, heads, kv, vocab, theta, seed):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=kv, vocab_size=vocab, rms_norm_eps=1e-5, rope_theta=theta,
                      tie_word_embeddings=False, attention_bias=False, mlp_bias=False, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    torch.manual_seed(seed)
    m = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for name, prm in m.named_parameters():
            if name.endswith("layernorm.weight") or name.endswith("norm.weight"):
                prm.copy_(1.0 + 0.1 * torch.randn_like(prm))           # norm weights away from one
            prm.data = prm.data.half()                                  # parameters to fp16; inv_freq stays fp32
    return m, cfg


def _params_from_hf(m, cfg):
    sd = m.state_dict()
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append({"q": sd[p + "self_attn.q_proj.weight"], "k": sd[p + "self_attn.k_proj.weight"],
                       "v": sd[p + "self_attn.v_proj.weight"], "o": sd[p + "self_attn.o_proj.weight"],
                       "gate": sd[p + "mlp.gate_proj.weight"], "up": sd[p + "mlp.up_proj.weight"],
                       "down": sd[p + "mlp.down_proj.weight"], "input_norm": sd[p + "input_layernorm.weight"],
                       "post_norm": sd[p + "post_attention_layernorm.weight"]})
    return {"embed": sd["model.embed_tokens.weight"], "layers": layers, "norm": sd["model.norm.weight"],
            "lm_head": sd["lm_head.weight"], "n_heads": cfg.num_attention_heads, "n_kv": cfg.num_key_value_heads,
            "head_dim": cfg.hidden_size // cfg.num_attention_heads, "eps": cfg.rms_norm_eps, "theta": 500000.0}


@pytest.mark.parametrize("shape", [
    # tiny: 2 layers, grouped-query 4:2
    dict(hidden=256, inter=512, layers=2, heads=4, kv=2, vocab=1024, tokens=24, batch=2),
    # two layers of the Llama-3-8B architecture (hidden 4096, 32 heads, 8 KV heads, intermediate 14336, theta 5e5)
    dict(hidden=4096, inter=14336, layers=2, heads=32, kv=8, vocab=2048, tokens=12, batch=1),
])
def test_model_oracle_matches_transformers_llama(shape):
    m, cfg = _hf_model(shape["hidden"], shape["inter"], shape["layers"], shape["heads"], shape["kv"], shape["vocab"],
                       500000.0, seed=0)
    params = _params_from_hf(m, cfg)
    ids = torch.randint(0, shape["vocab"], (shape["batch"], shape["tokens"]), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        hf = m(ids).logits.float()
        ours = llama_ref.forward(params, ids).float()
    err = ((hf - ours).abs().max() / hf.abs().max()).item()
    assert err <= TOL, err
    assert (hf.argmax(-1) == ours.argmax(-1)).float().mean().item() >= 0.95
