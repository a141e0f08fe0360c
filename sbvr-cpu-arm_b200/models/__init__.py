"""Llama on SBVR linears (`SBVRLinear`, `SBVRLlamaForCausalLM`) and the slicing helpers of its tensor-parallel form."""
