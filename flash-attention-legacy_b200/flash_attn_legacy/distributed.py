"""Multi-GPU use of the attention kernels: independent-unit sharding and a ring KV exchange.

The reference has no multi-GPU code at all (no NCCL, no torch.distributed); this module is
new surface.  One process per GPU, `torch.distributed` for the plumbing.

* `shard_range` / `shard_heads`: attention over different (batch, KV-head group) units is
  independent, so batched, packed and decode workloads are split across ranks with no
  communication on the data path.
* `ring_attention_forward` / `ring_attention_backward`: context parallelism for one very long
  sequence.  Rank r owns the contiguous rows [r*N/G, (r+1)*N/G) of q, k, v.  K/V shards travel
  around the ring with NCCL point-to-point send/recv on the side while the local kernels run
  on the shard already present; each step produces a partial (O, LSE) that is merged exactly
  (log-sum-exp algebra).  A shard that lies entirely in the causal future is skipped, the
  diagonal shard is causal, older shards are unmasked.  Received shards always land in this
  rank's own memory before a kernel reads them.

The compute steps are injected (`local_fwd`, `local_bwd`): on a GPU they are the library's
kernels, in the CPU tests they are the fp32 oracle, so the exchange logic is tested with the
gloo backend without a GPU.
"""
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(num_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, end) share of `num_units` independent units; sizes differ by at most 1."""
    base, extra = divmod(num_units, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_heads(heads_q: int, heads_kv: int, world_size: int, rank: int) -> Tuple[slice, slice]:
    """Splits by KV head so that every query head stays with the KV head it reads."""
    lo, hi = shard_range(heads_kv, world_size, rank)
    group = heads_q // heads_kv
    return slice(lo * group, hi * group), slice(lo, hi)


def merge_partials(o_acc: Optional[torch.Tensor], lse_acc: Optional[torch.Tensor],
                   o_part: torch.Tensor, lse_part: torch.Tensor):
    """Exact merge of two softmax partials over disjoint key sets.  O in fp32 [..., N, d], LSE [..., N]."""
    o_part = o_part.float()
    if o_acc is None:
        return o_part, lse_part.clone()
    lse_new = torch.logaddexp(lse_acc, lse_part)
    # rows that saw no key in either part keep -inf / zero
    w_acc = torch.exp(lse_acc - lse_new).nan_to_num(nan=0.0).unsqueeze(-1)
    w_part = torch.exp(lse_part - lse_new).nan_to_num(nan=0.0).unsqueeze(-1)
    return o_acc * w_acc + o_part * w_part, lse_new


def _exchange(send: List[torch.Tensor], recv: List[torch.Tensor], group, rank: int, world: int):
    """Posts the sends to the next rank and the receives from the previous one; returns requests."""
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    ops = []
    for t in send:
        ops.append(dist.P2POp(dist.isend, t, dist.get_global_rank(group, nxt) if group else nxt, group))
    for t in recv:
        ops.append(dist.P2POp(dist.irecv, t, dist.get_global_rank(group, prv) if group else prv, group))
    return dist.batch_isend_irecv(ops)


def _kernel_fwd(q, k, v, scale, causal):
    import flash_attn_legacy_cuda as ext
    return ext.forward_rect(q, k, v, scale, causal)


def _kernel_bwd(d_out, q, k, v, o, lse, scale, causal):
    import flash_attn_legacy_cuda as ext
    return ext.backward(d_out, q, k, v, o, lse, scale, causal)


def ring_attention_forward(q, k, v, softmax_scale: float, causal: bool = True, group=None,
                           local_fwd: Callable = _kernel_fwd):
    """Forward over a sequence sharded contiguously across the ranks of `group`.

    q [B,Hq,Nl,d], k/v [B,Hkv,Nl,d]: this rank's rows.  Returns (O [B,Hq,Nl,d] in q's dtype,
    LSE fp32 [B,Hq,Nl]) for this rank's rows, equal to attention over the whole sequence.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    k_nxt, v_nxt = torch.empty_like(k_cur), torch.empty_like(v_cur)
    o_acc, lse_acc = None, None
    for step in range(world):
        reqs = _exchange([k_cur, v_cur], [k_nxt, v_nxt], group, rank, world) if step + 1 < world else []
        src = (rank - step) % world  # owner of the shard held now
        if not (causal and src > rank):
            o_p, lse_p = local_fwd(q, k_cur, v_cur, softmax_scale, causal and src == rank)
            o_acc, lse_acc = merge_partials(o_acc, lse_acc, o_p, lse_p)
        for r in reqs:
            r.wait()
        k_cur, k_nxt = k_nxt, k_cur
        v_cur, v_nxt = v_nxt, v_cur
    return o_acc.to(q.dtype), lse_acc


def ring_attention_backward(d_out, q, k, v, o, lse, softmax_scale: float, causal: bool = True, group=None,
                            local_bwd: Callable = _kernel_bwd):
    """Backward of `ring_attention_forward`.  `o`, `lse` are its outputs for this rank's rows.

    dQ stays local (summed over the shards this rank's queries see, in fp32).  Each K/V shard
    travels the ring together with its fp32 dK/dV accumulator; after the last step one more hop
    returns the accumulator to the shard's owner.  Returns (dQ, dK, dV) for this rank's rows.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    k_nxt, v_nxt = torch.empty_like(k_cur), torch.empty_like(v_cur)
    dk_cur = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
    dv_cur = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
    dk_nxt, dv_nxt = torch.empty_like(dk_cur), torch.empty_like(dv_cur)
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    for step in range(world):
        # K/V of the next step can move while this step computes; the gradient accumulators
        # can only move once this step has added its share.
        kv_reqs = _exchange([k_cur, v_cur], [k_nxt, v_nxt], group, rank, world) if step + 1 < world else []
        src = (rank - step) % world
        if not (causal and src > rank):
            dq_p, dk_p, dv_p = local_bwd(d_out, q, k_cur, v_cur, o, lse, softmax_scale, causal and src == rank)
            dq += dq_p.float()
            dk_cur += dk_p.float()
            dv_cur += dv_p.float()
        for r in kv_reqs:
            r.wait()
        for r in _exchange([dk_cur, dv_cur], [dk_nxt, dv_nxt], group, rank, world):
            r.wait()
        k_cur, k_nxt = k_nxt, k_cur
        v_cur, v_nxt = v_nxt, v_cur
        dk_cur, dk_nxt = dk_nxt, dk_cur
        dv_cur, dv_nxt = dv_nxt, dv_cur
    # After `world` hops every accumulator is back at its owner.
    return dq.to(q.dtype), dk_cur.to(k.dtype), dv_cur.to(v.dtype)
