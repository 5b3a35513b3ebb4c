"""Autograd operators and modules: the Python operator surface of flash_attn_legacy on B200.

Drop-in for flash_attn_legacy/flash_attn.py of sirCamp/flash-attention-legacy:
`flash_attention`, `flash_attn_varlen_func`, `FlashAttentionFunc`,
`FlashAttnVarlenFunc`, `FlashAttention`, `FlashMultiHeadAttention` keep their
names, argument meaning, assertions and return conventions.  Added:
`flash_attn_with_kvcache` (single-token decode against a KV cache) -- the
reference has no such entry; its HF hook falls back to eager attention there.

All compute is in the sm_100a kernels reached through `flash_attn_legacy_cuda`.
"""
import math
from typing import Optional

import torch
import torch.nn as nn
from torch.autograd import Function

try:
    import flash_attn_legacy_cuda
except ImportError as e:  # same failure mode as the reference: no extension, no package
    raise ImportError(
        "flash_attn_legacy_cuda (the B200 attention library binding) could not be imported. "
        "Build it with: python flash-attention-legacy_b200/build.py\n"
        f"Original error: {e}"
    )

# Head dims of the reference (csrc/flash_attn_legacy.cpp:56).  64, 128 and 256 have kernels of their
# own; 32 and 96 run on the 64 / 128 kernels inside the library, which reads the missing columns as
# zeros through its TMA descriptors and never writes them -- no padded copies on this side.
SUPPORTED_HEAD_DIMS = (32, 64, 96, 128, 256)


def _kernel_ready(t: torch.Tensor) -> torch.Tensor:
    """`t` itself when the kernels can address it through strides, else a contiguous copy.

    The library takes (batch, head, row) element strides, so a [B,H,N,d] view of [B,N,H,d] memory
    (what a QKV projection followed by .transpose(1, 2) gives) needs no copy, where the reference
    copies every input (flash_attn.py:39).  Needed: head_dim contiguous, 16-byte aligned rows, and
    a real (positive) stride on every dimension longer than one -- an `expand`ed tensor (stride 0:
    K/V broadcast over heads, or the gradient of a `sum`) is copied.
    """
    if (t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all(s % 8 == 0 and (s > 0 or n == 1) for s, n in zip(t.stride()[:-1], t.shape[:-1]))):
        return t
    return t.contiguous()


class FlashAttentionFunc(Function):
    """q [B,Hq,N,d], k/v [B,Hkv,N,d] fp16 -> o [B,Hq,N,d]; Hq % Hkv == 0 (GQA / MQA).

    Mirrors FlashAttentionFunc of the reference (flash_attn.py:22-56).  `out_layout="bnhd"`
    (not in the reference) makes the result a [B,Hq,N,d] view of [B,N,Hq,d] memory, so that the
    `.transpose(1, 2)` a transformer block applies next is already contiguous.
    """

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, is_causal, out_layout="bhnd"):
        assert q.dtype == torch.float16, f"Q must be float16, got {q.dtype}"
        assert k.dtype == torch.float16 and v.dtype == torch.float16
        assert q.is_cuda and q.dim() == 4
        d = q.shape[-1]
        assert d in SUPPORTED_HEAD_DIMS, f"head_dim must be 32, 64, 96, 128, or 256, got {d}"
        h_q, h_kv = q.shape[1], k.shape[1]
        assert h_q % h_kv == 0, f"H_q ({h_q}) must be divisible by H_kv ({h_kv})"

        assert out_layout in ("bhnd", "bnhd"), f"out_layout must be 'bhnd' or 'bnhd', got {out_layout}"
        q, k, v = _kernel_ready(q), _kernel_ready(k), _kernel_ready(v)
        out = None
        if out_layout == "bnhd":
            b, _, n, _ = q.shape
            out = torch.empty((b, n, h_q, d), dtype=q.dtype, device=q.device).transpose(1, 2)
        o, lse = flash_attn_legacy_cuda.forward(q, k, v, softmax_scale, is_causal, out=out)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.softmax_scale = softmax_scale
        ctx.is_causal = is_causal
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = flash_attn_legacy_cuda.backward(
            _kernel_ready(grad_output), q, k, v, o, lse, ctx.softmax_scale, ctx.is_causal
        )
        return dq, dk, dv, None, None, None


def flash_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    is_causal: bool = False,
    out_layout: str = "bhnd",
) -> torch.Tensor:
    """softmax(q k^T * scale [+ causal mask]) v, O(N) memory, fp16 in / fp16 out.

    q [B,Hq,N,d]; k, v [B,Hkv,N,d] with Hq divisible by Hkv (MHA, GQA, MQA).
    `softmax_scale` defaults to 1/sqrt(d).  The causal mask hides key j from query i
    when j > i.  Same contract as the reference's flash_attention (flash_attn.py:59-87);
    inputs that are strided views with a contiguous head_dim are read in place, and
    `out_layout="bnhd"` returns the [B,Hq,N,d] result as a view of [B,N,Hq,d] memory.
    """
    assert q.dtype == torch.float16, f"Q must be float16, got {q.dtype}"
    d = q.shape[-1]
    assert d in SUPPORTED_HEAD_DIMS, f"head_dim must be 32, 64, 96, 128, or 256, got {d}"
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    return FlashAttentionFunc.apply(q, k, v, softmax_scale, is_causal, out_layout)


class FlashAttentionChunkFunc(Function):
    """Causal attention of the LAST Nq positions of a sequence against all its Nk keys (mask aligned to
    the end of the keys), with its backward.  Not in the reference, whose hook computes this case
    eagerly with a top-left mask (integrations.py:77-98)."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, out_layout="bhnd"):
        q, k, v = _kernel_ready(q), _kernel_ready(k), _kernel_ready(v)
        out = None
        if out_layout == "bnhd":
            b, h_q, n, d = q.shape
            out = torch.empty((b, n, h_q, d), dtype=q.dtype, device=q.device).transpose(1, 2)
        o, lse = flash_attn_legacy_cuda.forward_rect(q, k, v, softmax_scale, True, bottom_right=True, out=out)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.softmax_scale = softmax_scale
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = flash_attn_legacy_cuda.backward(
            _kernel_ready(grad_output), q, k, v, o, lse, ctx.softmax_scale, True, bottom_right=True
        )
        return dq, dk, dv, None, None


def flash_attention_chunk(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    out_layout: str = "bhnd",
) -> torch.Tensor:
    """Causal attention of a prompt chunk against a longer key sequence.

    q [B,Hq,Nq,d] holds the LAST Nq positions of the sequence whose keys and values are
    k, v [B,Hkv,Nk,d] with Nk >= Nq: query i sees keys j <= i + (Nk - Nq) (the causal mask is
    aligned to the bottom-right corner).  This is the step between prefill and single-token
    decode -- prefill in chunks, or a few new tokens after a cached prefix -- which the reference
    sends to its eager fallback with its usual top-left mask (integrations.py:63, :77-98).
    Not in the reference's API.  Differentiable.
    """
    assert q.dtype == torch.float16 and k.dtype == torch.float16 and v.dtype == torch.float16
    assert q.is_cuda and q.dim() == 4
    d = q.shape[-1]
    assert d in SUPPORTED_HEAD_DIMS, f"head_dim must be 32, 64, 96, 128, or 256, got {d}"
    assert q.shape[1] % k.shape[1] == 0, "H_q must be divisible by H_kv"
    assert k.shape[2] >= q.shape[2], "the key sequence must be at least as long as the query chunk"
    assert out_layout in ("bhnd", "bnhd"), f"out_layout must be 'bhnd' or 'bnhd', got {out_layout}"
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    return FlashAttentionChunkFunc.apply(q, k, v, softmax_scale, out_layout)


class FlashAttnVarlenFunc(Function):
    """Packed-sequence attention; forward AND backward are single native calls.

    Mirrors FlashAttnVarlenFunc of the reference (flash_attn.py:90-159); the reference's
    backward loops over sequences in Python with four host syncs each, this one does not.
    """

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                softmax_scale, is_causal, bottom_right=False):
        assert q.dtype == torch.float16, f"Q must be float16, got {q.dtype}"
        assert q.is_cuda and q.dim() == 3
        d = q.shape[-1]
        assert d in SUPPORTED_HEAD_DIMS, f"head_dim must be 32, 64, 96, 128, or 256, got {d}"

        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        cu_seqlens_q = cu_seqlens_q.contiguous().to(torch.int32)
        cu_seqlens_k = cu_seqlens_k.contiguous().to(torch.int32)
        o, lse = flash_attn_legacy_cuda.forward_varlen(
            q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, is_causal,
            bottom_right=bottom_right,
        )
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens_q, cu_seqlens_k)
        ctx.softmax_scale = softmax_scale
        ctx.is_causal = is_causal
        ctx.bottom_right = bottom_right
        ctx.max_seqlen_q = max_seqlen_q
        ctx.max_seqlen_k = max_seqlen_k
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = flash_attn_legacy_cuda.backward_varlen(
            grad_output.contiguous(), q, k, v, o, lse, cu_q, cu_k,
            ctx.max_seqlen_q, ctx.max_seqlen_k, ctx.softmax_scale, ctx.is_causal,
            bottom_right=ctx.bottom_right,
        )
        return dq, dk, dv, None, None, None, None, None, None, None


def flash_attn_varlen_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    causal_bottom_right: bool = False,
) -> torch.Tensor:
    """Attention over sequences packed along the token axis (no padding).

    q [total_q,H,d]; k, v [total_k,H_k,d]; cu_seqlens_* int32 [num_seqs+1] with the
    cumulative lengths.  Returns [total_q,H,d].  Same contract as the reference's
    flash_attn_varlen_func (flash_attn.py:162-220).  The causal mask is aligned to the
    top-left corner of each sequence's score matrix (key j hidden when j > i), as in
    the reference kernels (flash_attn_fwd_volta.cu:448-451).  `causal_bottom_right=True`
    (not in the reference) aligns it to the bottom-right corner instead: a sequence's queries
    are the last len_q positions of its len_k keys -- ragged chunks of new tokens behind
    ragged cached prefixes.
    """
    assert q.dim() == 3, f"q must be [total, heads, d], got shape {q.shape}"
    assert k.dim() == 3, f"k must be [total, heads_k, d], got shape {k.shape}"
    assert v.dim() == 3, f"v must be [total, heads_k, d], got shape {v.shape}"
    assert q.dtype == torch.float16, f"Q must be float16, got {q.dtype}"
    d = q.shape[-1]
    assert d in SUPPORTED_HEAD_DIMS, f"head_dim must be 32, 64, 96, 128, or 256, got {d}"
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    return FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                     softmax_scale, causal, causal_bottom_right)


def flash_attn_with_kvcache(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    k: Optional[torch.Tensor] = None,
    v: Optional[torch.Tensor] = None,
    cache_seqlens: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    cache_layout: str = "bshd",
    cache_starts: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention of new query tokens against key/value caches filled to a length per entry.

    q [B,Lq,Hq,d].  Caches are [B,S,Hkv,d] (`cache_layout="bshd"`) or [B,Hkv,S,d] ("bhsd",
    HuggingFace); entry b holds cache_seqlens[b] positions (from position cache_starts[b] on, if
    given: the positions before it are left padding -- decode only).  If k, v ([B,Lq,Hkv,d]) are
    given they are written into the caches at positions cache_seqlens[b] ... + Lq - 1 first and
    attended to as well; `cache_seqlens` itself is not modified.  Inference only.

    Lq == 1 is a decode step: no causal mask, as in the reference hook's decode branch
    (integrations.py:77-98), on the split-K kernel.  Lq > 1 is a chunk of a longer prompt: the
    chunk's tokens see the entry's cached positions and, causally, each other (the mask is aligned
    to the end of every entry's keys); it runs on the forward kernel with a key length per entry.
    The reference computes both cases eagerly over the whole cache.
    """
    assert q.dim() == 4, "q must be [B, L_q, H_q, d]"
    assert q.dtype == torch.float16, f"Q must be float16, got {q.dtype}"
    b, lq, hq, d = q.shape
    assert d in SUPPORTED_HEAD_DIMS, f"head_dim must be 32, 64, 96, 128, or 256, got {d}"
    seq_axis = 1 if cache_layout == "bshd" else 2
    if cache_seqlens is None:
        cache_seqlens = torch.full((b,), k_cache.shape[seq_axis], dtype=torch.int32, device=q.device)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    if lq == 1:
        k_new = k.reshape(b, -1, d).contiguous() if k is not None else None
        v_new = v.reshape(b, -1, d).contiguous() if v is not None else None
        out = flash_attn_legacy_cuda.decode(
            q.reshape(b, hq, d).contiguous(), k_cache, v_cache, cache_seqlens.to(torch.int32),
            softmax_scale, k_new, v_new, cache_layout=cache_layout,
            cache_starts=cache_starts.to(torch.int32).contiguous() if cache_starts is not None else None,
        )
        return out.view(b, 1, hq, d)

    assert cache_starts is None, "left-padded caches are supported for single-token steps only"
    lens = cache_seqlens.to(torch.int32)
    if k is not None:
        assert v is not None and k.shape == v.shape and k.shape[:2] == (b, lq), "k, v must be [B, L_q, H_kv, d]"
        # rows lens[b] ... lens[b] + Lq - 1 of every entry (an entry without room for the chunk is an error
        # the indexing reports)
        pos = lens.long()[:, None] + torch.arange(lq, device=q.device)[None, :]
        rows = torch.arange(b, device=q.device)[:, None]
        if cache_layout == "bshd":
            k_cache[rows, pos] = k
            v_cache[rows, pos] = v
        else:
            k_cache.transpose(1, 2)[rows, pos] = k
            v_cache.transpose(1, 2)[rows, pos] = v
        lens = lens + lq
    kc = k_cache.transpose(1, 2) if cache_layout == "bshd" else k_cache
    vc = v_cache.transpose(1, 2) if cache_layout == "bshd" else v_cache
    # O is written as [B,Lq,Hq,d] memory through its [B,Hq,Lq,d] view: no transpose afterwards
    out = torch.empty((b, lq, hq, d), dtype=torch.float16, device=q.device)
    flash_attn_legacy_cuda.forward_kvcache(q.transpose(1, 2), kc, vc, lens.contiguous(), softmax_scale, True,
                                           out=out.transpose(1, 2))
    return out


class FlashAttention(nn.Module):
    """Module form of flash_attention with a fixed head_dim, causal flag and scale."""

    def __init__(self, head_dim: int = 64, causal: bool = False,
                 softmax_scale: Optional[float] = None):
        super().__init__()
        assert head_dim in SUPPORTED_HEAD_DIMS
        self.head_dim = head_dim
        self.causal = causal
        self.softmax_scale = softmax_scale or (1.0 / math.sqrt(head_dim))

    def forward(self, q, k, v):
        return flash_attention(q, k, v, self.softmax_scale, self.causal)


class FlashMultiHeadAttention(nn.Module):
    """Multi-head attention block (q/k/v/out projections) on the flash kernels.

    `num_kv_heads` < `num_heads` gives GQA, 1 gives MQA.  Inputs in any float dtype are
    computed in fp16 and cast back; dropout is applied after the output projection.
    Same constructor and forward signature as the reference's module (flash_attn.py:238-312).
    """

    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: Optional[int] = None,
                 causal: bool = False, bias: bool = True, dropout: float = 0.0):
        super().__init__()
        num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        assert embed_dim % num_heads == 0
        assert num_heads % num_kv_heads == 0, (
            f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})"
        )
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = embed_dim // num_heads
        assert self.head_dim in SUPPORTED_HEAD_DIMS, (
            f"head_dim={self.head_dim}, must be 32, 64, 96, 128, or 256"
        )
        self.causal = causal
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.q_proj = nn.Linear(embed_dim, num_heads * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(embed_dim, num_kv_heads * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(embed_dim, num_kv_heads * self.head_dim, bias=bias)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x: torch.Tensor, key_value: Optional[torch.Tensor] = None):
        """x [B,N,embed_dim] (and optional key_value [B,N_kv,embed_dim]) -> [B,N,embed_dim]."""
        bsz, n, _ = x.shape
        src = x if key_value is None else key_value
        q = self.q_proj(x).view(bsz, n, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(src).view(bsz, -1, self.num_kv_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(src).view(bsz, -1, self.num_kv_heads, self.head_dim).transpose(1, 2)
        in_dtype = q.dtype
        if in_dtype != torch.float16:
            q, k, v = q.half(), k.half(), v.half()
        # q, k, v are [B,H,N,d] views of the projections' [B,N,H,d] memory and the result is written
        # as [B,N,H,d] memory: no copy on either side of the kernel (the reference copies all four).
        out = flash_attention(q, k, v, self.scale, self.causal, out_layout="bnhd")
        if in_dtype != torch.float16:
            out = out.to(in_dtype)
        out = out.transpose(1, 2).contiguous().view(bsz, n, self.embed_dim)  # already contiguous
        return self.dropout(self.out_proj(out))
