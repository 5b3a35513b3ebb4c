"""CPU oracle for the attention hot path -- TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this module; nothing under flash-attention-legacy_b200/ does.

It restates, in fp32 on the CPU, the math the reference library is checked
against by its own test-suite (sirCamp/flash-attention-legacy):

  attention_fwd      <- ref_attention,  tests/test_flash_attn.py:19-32
                        (GQA by repeat_interleave, scores * scale, strict upper
                        triangle -> -inf, softmax, P @ V); returns fp32 O, without
                        the reference's final .half(), plus the log-sum-exp whose
                        definition is pinned by csrc/kernels/flash_attn_fwd_volta.cu:343
                        (L = m + ln(l), natural log of the scaled masked scores).
  attention_bwd      <- ref_backward,   tests/test_flash_attn.py:35-58.  The reference
                        uses autograd; this is the closed form of the same
                        derivative (dV = P^T dO, dP = dO V^T, dS = P o (dP - rowsum(dO o O)),
                        dQ = scale dS K, dK = scale dS^T Q, GQA groups summed as at :56-57).
  varlen_fwd / _bwd  <- TestVarlen._ref_varlen, tests/test_flash_attn.py:293-308
                        (per-sequence loop over cu_seqlens).
  decode_fwd         <- the eager q_len != kv_len branch of the attention hook,
                        flash_attn_legacy/integrations.py:77-98 (GQA repeat, q k^T * scale,
                        softmax, @ v, no causal mask for q_len == 1), limited to the
                        first cache_seqlens[b] cache positions.

Parity pinned: tests/test_oracle.py checks every function here against
tests/golden/*.npz, which tests/golden/make_golden.py produced by running the
reference's own ref_attention / ref_backward / _ref_varlen and the reference's own
attention hook (decode branch) on seeded inputs.

The arithmetic is torch's CPU matmul / softmax, as in the reference's tests.
Large problems are processed in row blocks so that the score matrix fits in memory.
"""
import math

import torch


def _expand_kv(x, reps):
    return x if reps == 1 else x.repeat_interleave(reps, dim=1)


def _scores(q, k, scale, causal, causal_shift=0):
    """fp32 scaled scores [B,H,Nq,Nk] with the causal mask applied: key j is hidden from query i
    when j > i + causal_shift (0 = the reference's top-left-aligned mask)."""
    s = torch.matmul(q.float(), k.float().transpose(-2, -1)) * scale
    if causal:
        nq, nk = s.shape[-2], s.shape[-1]
        mask = torch.triu(torch.ones(nq, nk, dtype=torch.bool), diagonal=1 + causal_shift)
        s.masked_fill_(mask, float("-inf"))
    return s


def attention_fwd(q, k, v, scale, causal=False, causal_shift=0):
    """q [B,Hq,Nq,d], k/v [B,Hkv,Nk,d] (any float dtype) -> (O fp32 [B,Hq,Nq,d], LSE fp32 [B,Hq,Nq]).

    `causal_shift = Nk - Nq` gives the bottom-right-aligned mask of a chunk of new tokens behind a
    cached prefix: the same ref_attention arithmetic with the diagonal of its triu mask
    (tests/test_flash_attn.py:27-30) moved, so that the chunk's rows equal the last Nq rows of the
    square causal problem over all Nk positions (tests/test_oracle.py checks exactly that).
    """
    reps = q.shape[1] // k.shape[1]
    kf, vf = _expand_kv(k, reps), _expand_kv(v, reps)
    s = _scores(q, kf, scale, causal, causal_shift)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1).nan_to_num(nan=0.0)  # a row that sees no key: O = 0, LSE = -inf
    return torch.matmul(p, vf.float()), lse


def attention_bwd(q, k, v, d_out, scale, causal=False, causal_shift=0):
    """Closed-form gradients -> (dQ [B,Hq,Nq,d], dK [B,Hkv,Nk,d], dV [B,Hkv,Nk,d]) fp32.
    `causal_shift`: as in attention_fwd."""
    hq, hkv = q.shape[1], k.shape[1]
    reps = hq // hkv
    kf, vf = _expand_kv(k, reps).float(), _expand_kv(v, reps).float()
    qf, gf = q.float(), d_out.float()
    p = torch.softmax(_scores(q, kf, scale, causal, causal_shift), dim=-1).nan_to_num(nan=0.0)  # rows that see no key
    o = torch.matmul(p, vf)
    dv_full = torch.matmul(p.transpose(-2, -1), gf)
    dp = torch.matmul(gf, vf.transpose(-2, -1))
    delta = (gf * o).sum(dim=-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.matmul(ds, kf) * scale
    dk_full = torch.matmul(ds.transpose(-2, -1), qf) * scale
    b, _, nk, d = k.shape
    dk = dk_full.view(b, hkv, reps, nk, d).sum(dim=2)
    dv = dv_full.view(b, hkv, reps, nk, d).sum(dim=2)
    return dq, dk, dv


def _seq_bounds(cu):
    cu = [int(x) for x in cu]
    return list(zip(cu[:-1], cu[1:]))


def varlen_fwd(q, k, v, cu_q, cu_k, scale, causal=False, bottom_right=False):
    """Packed q [total_q,Hq,d], k/v [total_k,Hkv,d] -> (O fp32 [total_q,Hq,d], LSE fp32 [total_q,Hq]).
    `bottom_right`: each sequence's causal mask is aligned to the end of its keys (causal_shift =
    len_k - len_q per sequence) instead of the reference's top-left alignment."""
    outs, lses = [], []
    for (qs, qe), (ks, ke) in zip(_seq_bounds(cu_q), _seq_bounds(cu_k)):
        shift = (ke - ks) - (qe - qs) if bottom_right else 0
        qi = q[qs:qe].permute(1, 0, 2).unsqueeze(0)
        ki = k[ks:ke].permute(1, 0, 2).unsqueeze(0)
        vi = v[ks:ke].permute(1, 0, 2).unsqueeze(0)
        oi, li = attention_fwd(qi, ki, vi, scale, causal, shift)
        outs.append(oi.squeeze(0).permute(1, 0, 2))
        lses.append(li.squeeze(0).permute(1, 0))
    return torch.cat(outs, dim=0), torch.cat(lses, dim=0)


def varlen_bwd(q, k, v, d_out, cu_q, cu_k, scale, causal=False, bottom_right=False):
    dq = torch.zeros(q.shape, dtype=torch.float32)
    dk = torch.zeros(k.shape, dtype=torch.float32)
    dv = torch.zeros(v.shape, dtype=torch.float32)
    for (qs, qe), (ks, ke) in zip(_seq_bounds(cu_q), _seq_bounds(cu_k)):
        qi = q[qs:qe].permute(1, 0, 2).unsqueeze(0)
        ki = k[ks:ke].permute(1, 0, 2).unsqueeze(0)
        vi = v[ks:ke].permute(1, 0, 2).unsqueeze(0)
        gi = d_out[qs:qe].permute(1, 0, 2).unsqueeze(0)
        a, b, c = attention_bwd(qi, ki, vi, gi, scale, causal, (ke - ks) - (qe - qs) if bottom_right else 0)
        dq[qs:qe] = a.squeeze(0).permute(1, 0, 2)
        dk[ks:ke] = b.squeeze(0).permute(1, 0, 2)
        dv[ks:ke] = c.squeeze(0).permute(1, 0, 2)
    return dq, dk, dv


def decode_fwd(q, k_cache, v_cache, cache_seqlens, scale, cache_starts=None):
    """q [B,Hq,d]; caches [B,S,Hkv,d]; attends to the first cache_seqlens[b] positions, from
    position cache_starts[b] on when given (the hook's additive padding mask, integrations.py:88-89,
    for a left-padded batch: the keys it sets to -inf are a prefix of the cache).

    -> (O fp32 [B,Hq,d], LSE fp32 [B,Hq]).
    """
    bsz, hq, d = q.shape
    hkv = k_cache.shape[2]
    reps = hq // hkv
    o = torch.zeros(bsz, hq, d, dtype=torch.float32)
    lse = torch.full((bsz, hq), float("-inf"), dtype=torch.float32)
    for b in range(bsz):
        n = int(cache_seqlens[b])
        s0 = min(int(cache_starts[b]), n) if cache_starts is not None else 0
        if n - s0 == 0:
            continue
        kb = _expand_kv(k_cache[b, s0:n].permute(1, 0, 2).unsqueeze(0), reps).float()  # [1,Hq,n-s0,d]
        vb = _expand_kv(v_cache[b, s0:n].permute(1, 0, 2).unsqueeze(0), reps).float()
        qb = q[b].float().view(1, hq, 1, d)
        s = torch.matmul(qb, kb.transpose(-2, -1)) * scale
        lse[b] = torch.logsumexp(s, dim=-1).view(hq)
        o[b] = torch.matmul(torch.softmax(s, dim=-1), vb).view(hq, d)
    return o, lse


def kvcache_chunk_fwd(q, k_cache, v_cache, cache_seqlens, scale, causal=True):
    """q [B,Hq,Lq,d]; caches [B,Hkv,S,d]; entry b attends to its first cache_seqlens[b] cache rows, the
    causal mask aligned to the end of them (query i sees keys <= cache_seqlens[b] - Lq + i): the eager
    arithmetic of the reference hook's cache branch (integrations.py:80-98), per entry, with the mask
    where a chunk behind a cached prefix needs it.  Rows of the caches behind an entry's length are
    not read.  -> (O fp32 [B,Hq,Lq,d], LSE fp32 [B,Hq,Lq]).
    """
    bsz, hq, lq, d = q.shape
    o = torch.zeros(bsz, hq, lq, d, dtype=torch.float32)
    lse = torch.full((bsz, hq, lq), float("-inf"), dtype=torch.float32)
    for b in range(bsz):
        n = int(cache_seqlens[b])
        if n == 0:
            continue
        ob, lb = attention_fwd(q[b:b + 1], k_cache[b:b + 1, :, :n], v_cache[b:b + 1, :, :n], scale, causal,
                               causal_shift=n - lq)
        o[b], lse[b] = ob[0], lb[0]
    return o, lse


def attention_fwd_rows(q, k, v, scale, causal, row_start, row_end):
    """attention_fwd restricted to query rows [row_start, row_end) -- same arithmetic, bounded memory.

    Returns (O fp32 [B,Hq,rows,d], LSE fp32 [B,Hq,rows]).
    """
    reps = q.shape[1] // k.shape[1]
    nk = k.shape[2]
    hi = min(nk, row_end) if causal else nk  # keys beyond the last row are all masked
    kf, vf = _expand_kv(k[:, :, :hi], reps).float(), _expand_kv(v[:, :, :hi], reps).float()
    s = torch.matmul(q[:, :, row_start:row_end].float(), kf.transpose(-2, -1)) * scale
    if causal:
        rows = torch.arange(row_start, row_end).view(-1, 1)
        cols = torch.arange(hi).view(1, -1)
        s.masked_fill_(cols > rows, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    return torch.matmul(torch.softmax(s, dim=-1), vf), lse


def attention_fwd_blocked(q, k, v, scale, causal=False, block=1024):
    nq = q.shape[2]
    outs, lses = [], []
    for r0 in range(0, nq, block):
        o, l = attention_fwd_rows(q, k, v, scale, causal, r0, min(nq, r0 + block))
        outs.append(o)
        lses.append(l)
    return torch.cat(outs, dim=2), torch.cat(lses, dim=2)


def attention_bwd_blocked(q, k, v, d_out, scale, causal=False, block=1024):
    """attention_bwd in query-row blocks; dK/dV accumulated over blocks."""
    hq, hkv = q.shape[1], k.shape[1]
    reps = hq // hkv
    b, _, nk, d = k.shape
    nq = q.shape[2]
    dq = torch.empty(q.shape, dtype=torch.float32)
    dk = torch.zeros(b, hkv, nk, d, dtype=torch.float32)
    dv = torch.zeros(b, hkv, nk, d, dtype=torch.float32)
    for r0 in range(0, nq, block):
        r1 = min(nq, r0 + block)
        hi = min(nk, r1) if causal else nk
        kf, vf = _expand_kv(k[:, :, :hi], reps).float(), _expand_kv(v[:, :, :hi], reps).float()
        qf, gf = q[:, :, r0:r1].float(), d_out[:, :, r0:r1].float()
        s = torch.matmul(qf, kf.transpose(-2, -1)) * scale
        if causal:
            rows = torch.arange(r0, r1).view(-1, 1)
            cols = torch.arange(hi).view(1, -1)
            s.masked_fill_(cols > rows, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.matmul(p, vf)
        dp = torch.matmul(gf, vf.transpose(-2, -1))
        ds = p * (dp - (gf * o).sum(dim=-1, keepdim=True))
        dq[:, :, r0:r1] = torch.matmul(ds, kf) * scale
        dk[:, :, :hi] += (torch.matmul(ds.transpose(-2, -1), qf) * scale).view(b, hkv, reps, hi, d).sum(2)
        dv[:, :, :hi] += torch.matmul(p.transpose(-2, -1), gf).view(b, hkv, reps, hi, d).sum(2)
    return dq, dk, dv


# ---------------------------------------------------------------------------
# Error metrics used by every parity test.
# ---------------------------------------------------------------------------
TOL_O = 2e-3     # max|O - O_ref| / max|O_ref|
TOL_GRAD = 1e-2  # same ratio, for each of dQ, dK, dV
TOL_LSE = 1e-3   # max|LSE - LSE_ref|


def rel_max_err(x, ref):
    ref = ref.float()
    denom = ref.abs().max().item()
    err = (x.float().cpu() - ref).abs().max().item()
    return err / denom if denom > 0 else err


def abs_max_err(x, ref):
    x = x.float().cpu()
    ref = ref.float()
    both_inf = torch.isinf(x) & torch.isinf(ref) & (x.sign() == ref.sign())
    diff = torch.where(both_inf, torch.zeros_like(x), (x - ref).abs())
    return diff.max().item()


def default_scale(d):
    return 1.0 / math.sqrt(d)
