"""flash_attn_legacy on B200: FlashAttention-2 forward / backward / varlen / decode for sm_100a.

Same import surface as sirCamp/flash-attention-legacy (flash_attn_legacy/__init__.py:29-56):

    from flash_attn_legacy import flash_attention, flash_attn_varlen_func
    out = flash_attention(q, k, v, is_causal=True)          # q [B,Hq,N,d], k/v [B,Hkv,N,d] fp16

plus `flash_attn_with_kvcache` for single-token decode and `flash_attention_chunk` for a chunk
of new tokens against a longer cache.  Importing the package registers
the "flash_attn_legacy" attention implementation with HuggingFace transformers when it
is installed.
"""

__version__ = "0.5.0"

from .flash_attn import (
    FlashAttention,
    FlashMultiHeadAttention,
    flash_attention,
    flash_attention_chunk,
    flash_attn_varlen_func,
    flash_attn_with_kvcache,
)
from .integrations import register
from .utils import check_gpu_compatibility, get_device_info

__all__ = [
    "flash_attention",
    "flash_attn_varlen_func",
    "flash_attn_with_kvcache",
    "flash_attention_chunk",
    "FlashAttention",
    "FlashMultiHeadAttention",
    "check_gpu_compatibility",
    "get_device_info",
    "register",
]

register()
