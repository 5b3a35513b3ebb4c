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
* `layout="zigzag"`: contiguous shards leave rank r with r+1 shard pairs under a causal mask, so
  the last rank sets the time.  In the zigzag layout the sequence is cut into 2G chunks and rank
  r owns chunks r and 2G-1-r (`zigzag_rows`); every rank then does the same work in every ring
  step: the diagonal step is one causal call over its two chunks, a shard from an earlier rank
  is read by all local queries but only its first chunk, a shard from a later rank is read in
  full but only by the second local chunk.

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


def zigzag_rows(seqlen: int, world_size: int, rank: int) -> Tuple[Tuple[int, int], Tuple[int, int]]:
    """Row ranges [start, end) of the two chunks rank `rank` owns in the zigzag layout.

    `seqlen` must be a multiple of 2 * world_size.  The rank's local tensor is the early chunk
    followed by the late chunk.
    """
    if seqlen % (2 * world_size):
        raise ValueError("zigzag layout needs seqlen divisible by 2 * world_size")
    c = seqlen // (2 * world_size)
    late = 2 * world_size - 1 - rank
    return (rank * c, (rank + 1) * c), (late * c, (late + 1) * c)


def zigzag_take(x: torch.Tensor, world_size: int, rank: int, dim: int = 2) -> torch.Tensor:
    """This rank's rows of a full-sequence tensor in the zigzag layout (a copy)."""
    (a0, a1), (b0, b1) = zigzag_rows(x.shape[dim], world_size, rank)
    return torch.cat([x.narrow(dim, a0, a1 - a0), x.narrow(dim, b0, b1 - b0)], dim)


def _merge_into(o_acc, lse_acc, rows: slice, o_part, lse_part):
    """In-place `merge_partials` restricted to the rows `rows` of the accumulators."""
    o_new, lse_new = merge_partials(o_acc[:, :, rows], lse_acc[:, :, rows], o_part, lse_part)
    o_acc[:, :, rows] = o_new
    lse_acc[:, :, rows] = lse_new


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


class _ShardRing:
    """The K/V (or any) shards a rank holds while they travel the ring.

    `cur` starts as the caller's own tensors, which are only ever sent; shards received later
    land alternately in two private buffers, so the caller's tensors are never written.
    """

    def __init__(self, tensors, group, rank: int, world: int):
        self.cur = [t.contiguous() for t in tensors]
        self._bufs = [None, None]
        self._turn = 0
        self._group, self._rank, self._world = group, rank, world
        self._incoming = None

    def start(self):
        """Posts send of `cur` to the next rank and receive of the previous rank's shards."""
        if self._bufs[self._turn] is None:
            self._bufs[self._turn] = [torch.empty_like(t) for t in self.cur]
        self._incoming = self._bufs[self._turn]
        return _exchange(self.cur, self._incoming, self._group, self._rank, self._world)

    def finish(self, reqs):
        """Waits for the posted exchange and makes the received shards current."""
        for r in reqs:
            r.wait()
        if self._incoming is not None:
            self.cur = self._incoming
            self._incoming = None
            self._turn ^= 1


def _kernel_fwd(q, k, v, scale, causal):
    import flash_attn_legacy_cuda as ext
    return ext.forward_rect(q, k, v, scale, causal)


def _kernel_bwd(d_out, q, k, v, o, lse, scale, causal):
    import flash_attn_legacy_cuda as ext
    return ext.backward(d_out, q, k, v, o, lse, scale, causal)


def _check_layout(layout: str, causal: bool, rows: int):
    if layout not in ("contiguous", "zigzag"):
        raise ValueError("layout must be 'contiguous' or 'zigzag'")
    if layout == "zigzag" and rows % 2:
        raise ValueError("zigzag layout needs an even number of local rows")
    # Without a mask every shard pair is full work on every rank: the two layouts coincide.
    return layout == "zigzag" and causal


def _shard_plan(zigzag: bool, causal: bool, rank: int, src: int, rows: int):
    """What this rank computes against the shard owned by `src`.

    Returns None (nothing to do) or (query rows, key rows, causal flag) with the row sets as
    slices into the local tensors.
    """
    everything = slice(0, rows)
    if not causal:
        return everything, everything, False
    if src == rank:
        # zigzag: the chunks [r, 2G-1-r] against themselves are causal over their concatenation
        return everything, everything, True
    if not zigzag:
        return (everything, everything, False) if src < rank else None
    c = rows // 2
    if src < rank:
        # its early chunk precedes both local chunks, its late chunk follows both
        return everything, slice(0, c), False
    # a later rank: both its chunks lie between the local early and late chunk
    return slice(c, rows), everything, False


def ring_attention_forward(q, k, v, softmax_scale: float, causal: bool = True, group=None,
                           local_fwd: Callable = _kernel_fwd, layout: str = "contiguous"):
    """Forward over a sequence sharded across the ranks of `group`.

    q [B,Hq,Nl,d], k/v [B,Hkv,Nl,d]: this rank's rows (contiguous shard, or its two zigzag chunks
    back to back).  Returns (O [B,Hq,Nl,d] in q's dtype, LSE fp32 [B,Hq,Nl]) for this rank's
    rows, equal to attention over the whole sequence.  The inputs are not modified.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    zigzag = _check_layout(layout, causal, q.shape[2])
    rows = q.shape[2]
    kv = _ShardRing([k, v], group, rank, world)
    o_acc, lse_acc = None, None
    for step in range(world):
        reqs = kv.start() if step + 1 < world else []
        plan = _shard_plan(zigzag, causal, rank, (rank - step) % world, rows)
        if plan is not None:
            qs, ks, masked = plan
            k_cur, v_cur = kv.cur
            o_p, lse_p = local_fwd(q[:, :, qs], k_cur[:, :, ks], v_cur[:, :, ks], softmax_scale, masked)
            if o_acc is None:  # step 0 is the diagonal and covers every local row
                o_acc, lse_acc = o_p.float(), lse_p.clone()
            elif qs.stop - qs.start == rows:
                o_acc, lse_acc = merge_partials(o_acc, lse_acc, o_p, lse_p)
            else:
                _merge_into(o_acc, lse_acc, qs, o_p, lse_p)
        kv.finish(reqs)
    return o_acc.to(q.dtype), lse_acc


def ring_attention_backward(d_out, q, k, v, o, lse, softmax_scale: float, causal: bool = True, group=None,
                            local_bwd: Callable = _kernel_bwd, layout: str = "contiguous"):
    """Backward of `ring_attention_forward`.  `o`, `lse` are its outputs for this rank's rows.

    dQ stays local (summed over the shards this rank's queries see, in fp32).  Each K/V shard
    travels the ring together with its fp32 dK/dV accumulator; after the last step one more hop
    returns the accumulator to the shard's owner.  Returns (dQ, dK, dV) for this rank's rows.
    The inputs are not modified.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    zigzag = _check_layout(layout, causal, q.shape[2])
    rows = q.shape[2]
    kv = _ShardRing([k, v], group, rank, world)
    grads = _ShardRing([torch.zeros(k.shape, dtype=torch.float32, device=k.device),
                        torch.zeros(v.shape, dtype=torch.float32, device=v.device)], group, rank, world)
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse_late = None
    grads_in_flight = None
    for step in range(world):
        # K/V of the next step move while this step computes.  The gradient accumulators of the
        # shard held now were sent by the previous rank after ITS previous step: that transfer is
        # left in flight during this step's kernels and only waited for when their result is added.
        kv_reqs = kv.start() if step + 1 < world else []
        plan = _shard_plan(zigzag, causal, rank, (rank - step) % world, rows)
        partial = None
        if plan is not None:
            qs, ks, masked = plan
            k_cur, v_cur = kv.cur
            if qs.stop - qs.start == rows:
                lse_rows = lse
            else:
                if lse_late is None:
                    lse_late = lse[:, :, qs].contiguous()
                lse_rows = lse_late
            partial = local_bwd(d_out[:, :, qs], q[:, :, qs], k_cur[:, :, ks], v_cur[:, :, ks],
                                o[:, :, qs], lse_rows, softmax_scale, masked)
        if grads_in_flight is not None:
            grads.finish(grads_in_flight)
        if partial is not None:
            dq_p, dk_p, dv_p = partial
            dk_cur, dv_cur = grads.cur
            dq[:, :, qs] += dq_p
            dk_cur[:, :, ks] += dk_p
            dv_cur[:, :, ks] += dv_p
        kv.finish(kv_reqs)
        grads_in_flight = grads.start()
    grads.finish(grads_in_flight)
    # After `world` hops every accumulator is back at its owner.
    dk_own, dv_own = grads.cur
    return dq.to(q.dtype), dk_own.to(k.dtype), dv_own.to(v.dtype)
