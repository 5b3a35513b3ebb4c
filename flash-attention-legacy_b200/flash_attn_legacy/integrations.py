"""HuggingFace Transformers hook: attn_implementation="flash_attn_legacy".

Drop-in for flash_attn_legacy/integrations.py of sirCamp/flash-attention-legacy:
`flash_attn_legacy_forward` has the AttentionInterface signature and returns
(attn_output [B,N,H,d], None); `register()` adds it to ALL_ATTENTION_FUNCTIONS and
patches PreTrainedModel._check_and_adjust_attn_implementation exactly where the
reference does (integrations.py:106-161).

Routing differs from the reference in two places.  Single-token decode without a mask
(or with the padding mask of a left-padded batch) goes to the split-K decode kernel instead of
eager matmul/softmax.  And a padding mask is
honoured: `register()` also registers transformers' 2-D ("which tokens are real") mask
format for this name -- without that, transformers hands a custom attention function no
mask at all, and the reference attends to padding (integrations.py:63-76) -- and a prefill
with such a mask runs un-padded through the packed kernels.  Everything the kernels do not
cover (an additive 4-D mask, a padding mask outside prefill, unsupported head_dim) keeps the
reference's eager arithmetic.  A third difference: several new tokens against a longer cache
(q_len > 1, kv_len > q_len, causal, no mask) run through the kernels (forward and backward) with
the causal mask aligned to the END of the key sequence -- the new tokens are its last q_len
positions -- where the reference's fallback applies its top-left mask (integrations.py:91-96),
which hides the cached prefix from the first new tokens.  The eager fallback here aligns its
mask the same way, so the result does not depend on which path a call takes.
"""
import math
from typing import Optional

import torch
import torch.nn as nn

_KERNEL_HEAD_DIMS = (32, 64, 96, 128, 256)
_DECODE_HEAD_DIMS = _KERNEL_HEAD_DIMS  # decode and chunked prefill cover the same head dims


def _resolve_causal(module, attention_mask, q_len, kwargs):
    # Same precedence as the reference (integrations.py:54-61): explicit kwarg, then the
    # module's flag, then "causal unless a mask was given or this is a single token".
    if "is_causal" in kwargs:
        return kwargs["is_causal"]
    if hasattr(module, "is_causal"):
        return module.is_causal
    return attention_mask is None and q_len > 1


def _eager_attention(query, key, value, attention_mask, scaling, is_causal):
    """The reference's fallback arithmetic (integrations.py:80-98), in the model dtype, with the
    causal mask aligned to the end of the key sequence."""
    h_q, h_kv = query.shape[1], key.shape[1]
    if h_kv != h_q:
        key = key.repeat_interleave(h_q // h_kv, dim=1)
        value = value.repeat_interleave(h_q // h_kv, dim=1)
    scores = torch.matmul(query, key.transpose(-2, -1)) * scaling
    if attention_mask is not None:
        scores = scores + attention_mask
    q_len, kv_len = query.shape[2], key.shape[2]
    if is_causal and q_len > 1:
        # The queries are the last q_len positions of the key sequence.  (The reference's triu has
        # diagonal=1 here, integrations.py:91-96: the same thing for q_len == kv_len, but behind a
        # cached prefix it hides the prefix from the first new tokens.)
        scores = scores + torch.triu(
            torch.full((q_len, kv_len), float("-inf"), device=query.device, dtype=query.dtype),
            diagonal=1 + kv_len - q_len,
        )
    return torch.matmul(torch.softmax(scores, dim=-1), value)


def _left_padding_starts(keep):
    """First real position of every row of `keep` [B, N] bool, as int32 [B], if the padding of every
    row is a prefix (what generation with a decoder-only model uses); None for any other pattern.
    Reads one flag back from the device."""
    n = keep.shape[1]
    starts = (n - keep.sum(dim=1)).to(torch.int32)
    prefix = torch.arange(n, device=keep.device)[None, :] >= starts[:, None]
    return starts if bool((keep == prefix).all()) else None


def _padded_prefill(query, key, value, keep, scaling, is_causal):
    """Prefill of a padded batch through the packed kernels.

    `keep` [B, N] bool marks the real tokens of every row (left or right padding, any pattern).
    Real tokens are packed in order, attend among themselves (causal order is preserved by the
    packing), and their outputs go back to their places; padded positions give zeros.
    Returns [B, N, Hq, d].
    """
    from .flash_attn import flash_attn_varlen_func

    bsz, h_q, n, d = query.shape
    h_kv = key.shape[1]
    idx = keep.reshape(-1).nonzero(as_tuple=True)[0]  # the un-padding; sizes depend on the data
    lens = keep.sum(dim=1, dtype=torch.int32)
    cu = torch.zeros(bsz + 1, dtype=torch.int32, device=query.device)
    cu[1:] = torch.cumsum(lens, dim=0)

    def pack(t, h):
        return t.transpose(1, 2).reshape(bsz * n, h, d).index_select(0, idx)

    out_packed = flash_attn_varlen_func(pack(query, h_q), pack(key, h_kv), pack(value, h_kv),
                                        cu, cu, n, n, softmax_scale=scaling, causal=is_causal)
    out = torch.zeros(bsz * n, h_q, d, dtype=out_packed.dtype, device=query.device)
    out.index_copy_(0, idx, out_packed)
    return out.view(bsz, n, h_q, d)


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
    from .flash_attn import flash_attention, flash_attention_chunk, flash_attn_with_kvcache

    bsz, h_q, q_len, d = query.shape
    kv_len = key.shape[2]
    if scaling is None:
        scaling = 1.0 / math.sqrt(d)
    # A 2-D mask says which key positions are real tokens (transformers' format for un-padded
    # attention, registered for this name by register()); anything else is additive.
    keep = None
    if attention_mask is not None and attention_mask.dim() == 2:
        keep = attention_mask.to(torch.bool)
        attention_mask = None
        if keep.shape[-1] != kv_len or bool(keep.all()):
            keep = None
    is_causal = _resolve_causal(module, attention_mask, q_len, kwargs)
    in_dtype = query.dtype

    def to_half(t):
        return t if t.dtype == torch.float16 else t.half()

    kernel_ok = d in _KERNEL_HEAD_DIMS and query.is_cuda
    if keep is not None and q_len == kv_len and kernel_ok:
        out = _padded_prefill(to_half(query), to_half(key), to_half(value), keep, scaling,
                              is_causal).to(in_dtype)
    elif (keep is not None and q_len == 1 and d in _DECODE_HEAD_DIMS and query.is_cuda
          and (starts := _left_padding_starts(keep)) is not None):
        # Decode of a left-padded batch: every entry skips its padded prefix of the cache.
        out = flash_attn_with_kvcache(
            to_half(query).transpose(1, 2), to_half(key), to_half(value),
            softmax_scale=scaling, cache_layout="bhsd", cache_starts=starts,
        ).to(in_dtype)
    elif keep is not None:
        # Other padding outside prefill: eager arithmetic with the
        # padded keys masked out; causal rows are aligned to the end of the key sequence.
        additive = torch.zeros(bsz, 1, q_len, kv_len, dtype=query.dtype, device=query.device)
        additive.masked_fill_(~keep[:, None, None, :], float("-inf"))
        if is_causal and q_len > 1:
            qi = torch.arange(q_len, device=query.device)[:, None] + (kv_len - q_len)
            kj = torch.arange(kv_len, device=query.device)[None, :]
            additive.masked_fill_((kj > qi)[None, None], float("-inf"))
        out = _eager_attention(query, key, value, additive, scaling, False)
        out = torch.nan_to_num(out).transpose(1, 2).contiguous()  # rows that see no key at all
    elif q_len == kv_len and kernel_ok:
        # Prefill.  As in the reference, attention_mask is not consulted on this branch.
        # Inputs are read through their strides and the result is written as [B, q_len, Hq, d]
        # memory, so neither side of the call copies (the reference copies q, k, v and the output:
        # flash_attn.py:39, integrations.py:101).
        out = flash_attention(to_half(query), to_half(key), to_half(value),
                              softmax_scale=scaling, is_causal=is_causal, out_layout="bnhd")
        out = out.to(in_dtype).transpose(1, 2).contiguous()  # no-op for fp16 models
    elif 1 < q_len < kv_len and attention_mask is None and is_causal and query.is_cuda and d in _DECODE_HEAD_DIMS:
        # A chunk of new tokens against a cache that holds earlier ones.
        out = flash_attention_chunk(to_half(query), to_half(key), to_half(value),
                                    softmax_scale=scaling, out_layout="bnhd")
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
        try:  # the mask format of un-padded attention: a 2-D "real token" mask, or None
            from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS, flash_attention_mask

            ALL_MASK_ATTENTION_FUNCTIONS.register("flash_attn_legacy", flash_attention_mask)
        except (ImportError, AttributeError):
            pass  # older transformers: no mask interface, the hook gets no mask as before
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
