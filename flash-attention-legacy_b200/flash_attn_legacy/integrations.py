"""HuggingFace Transformers hook: attn_implementation="flash_attn_legacy".

Drop-in for flash_attn_legacy/integrations.py of sirCamp/flash-attention-legacy:
`flash_attn_legacy_forward` has the AttentionInterface signature and returns
(attn_output [B,N,H,d], None); `register()` adds it to ALL_ATTENTION_FUNCTIONS and
patches PreTrainedModel._check_and_adjust_attn_implementation exactly where the
reference does (integrations.py:106-161).

Routing differs from the reference in one place: single-token decode without an
additive mask goes to the split-K decode kernel instead of eager matmul/softmax.
Everything the kernels do not cover (an explicit attention_mask, q_len > 1 with a
longer key sequence, unsupported head_dim) keeps the reference's eager arithmetic.
"""
import math
from typing import Optional

import torch
import torch.nn as nn

_KERNEL_HEAD_DIMS = (32, 64, 96, 128)
_DECODE_HEAD_DIMS = (64, 128)


def _resolve_causal(module, attention_mask, q_len, kwargs):
    # Same precedence as the reference (integrations.py:54-61): explicit kwarg, then the
    # module's flag, then "causal unless a mask was given or this is a single token".
    if "is_causal" in kwargs:
        return kwargs["is_causal"]
    if hasattr(module, "is_causal"):
        return module.is_causal
    return attention_mask is None and q_len > 1


def _eager_attention(query, key, value, attention_mask, scaling, is_causal):
    """The reference's fallback arithmetic (integrations.py:80-98), in the model dtype."""
    h_q, h_kv = query.shape[1], key.shape[1]
    if h_kv != h_q:
        key = key.repeat_interleave(h_q // h_kv, dim=1)
        value = value.repeat_interleave(h_q // h_kv, dim=1)
    scores = torch.matmul(query, key.transpose(-2, -1)) * scaling
    if attention_mask is not None:
        scores = scores + attention_mask
    q_len, kv_len = query.shape[2], key.shape[2]
    if is_causal and q_len > 1:
        scores = scores + torch.triu(
            torch.full((q_len, kv_len), float("-inf"), device=query.device, dtype=query.dtype),
            diagonal=1,
        )
    return torch.matmul(torch.softmax(scores, dim=-1), value)


def flash_attn_legacy_forward(
    module: nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    dropout: float = 0.0,
    scaling: Optional[float] = None,
    **kwargs,
):
    """query [B,Hq,q_len,d], key/value [B,Hkv,kv_len,d] -> (attn_output [B,q_len,Hq,d], None)."""
    from .flash_attn import flash_attention, flash_attn_with_kvcache

    bsz, h_q, q_len, d = query.shape
    kv_len = key.shape[2]
    if scaling is None:
        scaling = 1.0 / math.sqrt(d)
    is_causal = _resolve_causal(module, attention_mask, q_len, kwargs)
    in_dtype = query.dtype

    def to_half(t):
        return t if t.dtype == torch.float16 else t.half()

    if q_len == kv_len and d in _KERNEL_HEAD_DIMS and query.is_cuda:
        # Prefill.  As in the reference, attention_mask is not consulted on this branch.
        # Inputs are read through their strides and the result is written as [B, q_len, Hq, d]
        # memory, so neither side of the call copies (the reference copies q, k, v and the output:
        # flash_attn.py:39, integrations.py:101).
        out = flash_attention(to_half(query), to_half(key), to_half(value),
                              softmax_scale=scaling, is_causal=is_causal, out_layout="bnhd")
        out = out.to(in_dtype).transpose(1, 2).contiguous()  # no-op for fp16 models
    elif q_len == 1 and attention_mask is None and d in _DECODE_HEAD_DIMS and query.is_cuda:
        # Decode: one new token against the whole cache, no mask.
        out = flash_attn_with_kvcache(
            to_half(query).transpose(1, 2), to_half(key), to_half(value),
            softmax_scale=scaling, cache_layout="bhsd",
        ).to(in_dtype)  # already [B, 1, Hq, d]
    else:
        out = _eager_attention(query, key, value, attention_mask, scaling, is_causal)
        out = out.transpose(1, 2).contiguous()
    return out, None


def register():
    """Registers "flash_attn_legacy" with transformers; returns False if that is impossible.

    Two steps, as in the reference: (1) ALL_ATTENTION_FUNCTIONS.register(name, fn);
    (2) wrap PreTrainedModel._check_and_adjust_attn_implementation so that this name is
    accepted as-is -- transformers would otherwise treat any name containing "flash" as
    a request for the flash_attn package or a hub kernel and try to import one -- and so
    that a model whose head_dim the kernels do not cover is switched to "sdpa".
    """
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS, PreTrainedModel

        ALL_ATTENTION_FUNCTIONS.register("flash_attn_legacy", flash_attn_legacy_forward)
        stock_check = PreTrainedModel._check_and_adjust_attn_implementation
        if getattr(stock_check, "_flash_attn_legacy_patched", False):
            return True  # idempotent: do not stack wrappers on repeated imports

        def _check(self, attn_implementation, is_init_check=False, allow_all_kernels=False):
            if attn_implementation != "flash_attn_legacy":
                return stock_check(self, attn_implementation, is_init_check, allow_all_kernels)
            head_dim = getattr(self.config, "head_dim", None)
            if head_dim is None:
                hidden = getattr(self.config, "hidden_size", None)
                heads = getattr(self.config, "num_attention_heads", None)
                if hidden and heads:
                    head_dim = hidden // heads
            if head_dim is not None and head_dim not in (32, 64, 96, 128, 256):
                return stock_check(self, "sdpa", is_init_check, allow_all_kernels)
            return "flash_attn_legacy"

        _check._flash_attn_legacy_patched = True
        PreTrainedModel._check_and_adjust_attn_implementation = _check
        return True
    except (ImportError, AttributeError):
        return False
