"""LLaMA attention layers switched to the B200 kernels by replacing their `forward`.

Second integration route of sirCamp/flash-attention-legacy (examples/hf_llama_patch.py:19-125),
for transformers versions or model classes where `attn_implementation="flash_attn_legacy"`
cannot be used: every LlamaAttention module gets a new bound `forward` that does the layer's
own projections, rotary embedding and cache update and then calls the attention hook of this
package.  The hook picks the kernel -- prefill, single-token decode against the cache (split-K
kernel; the reference computes this step with eager matmul/softmax, :95-103), or a chunk of new
tokens behind a cached prefix -- so both routes share one code path and one set of tests.

    from hf_llama_patch import patch_llama_attention
    model = patch_llama_attention(AutoModelForCausalLM.from_pretrained(..., torch_dtype=torch.float16).cuda())
"""
import math

import torch

_PATCHED_CLASSES = ("LlamaAttention", "LlamaSdpaAttention", "LlamaFlashAttention2")


def _layer_geometry(attn):
    """(num_heads, num_kv_heads, head_dim) from the module (transformers < 5) or its config."""
    cfg = getattr(attn, "config", None)
    heads = getattr(attn, "num_heads", None) or cfg.num_attention_heads
    kv_heads = getattr(attn, "num_key_value_heads", None) or cfg.num_key_value_heads
    head_dim = getattr(attn, "head_dim", None) or cfg.hidden_size // heads
    return heads, kv_heads, head_dim


def _patched_forward(attn):
    from flash_attn_legacy.integrations import flash_attn_legacy_forward

    def forward(hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None,
                past_key_value=None, position_ids=None, use_cache=False, **kwargs):
        bsz, q_len, _ = hidden_states.shape
        heads, kv_heads, head_dim = _layer_geometry(attn)
        # [B, N, H*d] -> [B, H, N, d] views; the kernels read them through their strides
        q = attn.q_proj(hidden_states).view(bsz, q_len, heads, head_dim).transpose(1, 2)
        k = attn.k_proj(hidden_states).view(bsz, q_len, kv_heads, head_dim).transpose(1, 2)
        v = attn.v_proj(hidden_states).view(bsz, q_len, kv_heads, head_dim).transpose(1, 2)

        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
        if position_embeddings is not None:          # transformers >= 4.46 hands cos/sin down
            cos, sin = position_embeddings
            q, k = apply_rotary_pos_emb(q, k, cos, sin)
        elif hasattr(attn, "rotary_emb"):            # older: the layer owns the rotary module
            cos, sin = attn.rotary_emb(v, position_ids)
            q, k = apply_rotary_pos_emb(q, k, cos, sin)

        cache = past_key_values if past_key_values is not None else past_key_value
        if cache is not None and hasattr(cache, "update"):   # Cache object
            k, v = cache.update(k, v, attn.layer_idx)
        elif cache is not None:                              # legacy (k, v) tuple
            k = torch.cat([cache[0], k], dim=2)
            v = torch.cat([cache[1], v], dim=2)

        # As in the reference's patch, the mask argument is not consulted: the layer is causal.
        out, _ = flash_attn_legacy_forward(attn, q, k, v, None, scaling=1.0 / math.sqrt(head_dim),
                                           is_causal=q_len > 1)
        out = attn.o_proj(out.reshape(bsz, q_len, heads * head_dim))
        return out, None

    return forward


def patch_llama_attention(model):
    """Replaces the forward of every LLaMA attention layer of `model`; returns `model`."""
    patched = 0
    for module in model.modules():
        if module.__class__.__name__ in _PATCHED_CLASSES:
            module.forward = _patched_forward(module)
            patched += 1
    print(f"Patched {patched} attention layers with flash_attn_legacy")
    return model


def main():
    import argparse

    from transformers import AutoModelForCausalLM, AutoTokenizer

    from flash_attn_legacy import check_gpu_compatibility

    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="meta-llama/Llama-2-7b-hf")
    ap.add_argument("--prompt", default="The meaning of life is")
    ap.add_argument("--max-new-tokens", type=int, default=50)
    args = ap.parse_args()
    check_gpu_compatibility()
    tok = AutoTokenizer.from_pretrained(args.model)
    model = AutoModelForCausalLM.from_pretrained(args.model, torch_dtype=torch.float16, device_map="cuda")
    patch_llama_attention(model)
    inputs = tok(args.prompt, return_tensors="pt").to("cuda")
    with torch.no_grad():
        out = model.generate(**inputs, max_new_tokens=args.max_new_tokens, do_sample=True, temperature=0.7)
    print(tok.decode(out[0], skip_special_tokens=True))


if __name__ == "__main__":
    main()
