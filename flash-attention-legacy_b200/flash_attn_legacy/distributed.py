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

Between the attention kernels of a ring step runs ONE small kernel and no tensor arithmetic of
the framework: the forward merges each partial (O, LSE) into fp32 accumulators with the library's
merge kernel; the backward lets the kernel add dQ into an fp32 accumulator that lives for the
whole pass, takes dK/dV as unrounded fp32 partials and adds them to the accumulators that travel
with their shard.  Every gradient is therefore rounded to fp16 exactly once, at the end, whatever
the number of ranks.

The compute steps are injected (`steps`): on a GPU they are the library's kernels
(`KernelSteps`), in the CPU tests they are the fp32 oracle, so the exchange logic is tested
with the gloo backend without a GPU.

Failure detection (host side): every rank checks at entry that all ranks hold shards of one
shape (`RingShardError` on every rank otherwise, before any data moves), and a wait for a
neighbour's shard can be given a time limit (`timeout_s`): when it runs out -- a neighbour left
between steps -- the call raises `RingTimeoutError` instead of blocking.  The limit is enforced
by the backend's timed wait for CPU tensors (gloo); for CUDA tensors the wait is a stream dependency
that never blocks the host, and a neighbour that has gone is reported by the process group's own
timeout on the next collective.
"""
import datetime
import time
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


class RingShardError(ValueError):
    """The ranks of a ring do not hold shards of one shape."""


class RingTimeoutError(RuntimeError):
    """A neighbour's shard did not arrive within the time limit."""


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


def merge_partials(o_acc: Optional[torch.Tensor], lse_acc: Optional[torch.Tensor],
                   o_part: torch.Tensor, lse_part: torch.Tensor):
    """Exact merge of two softmax partials over disjoint key sets.  O in fp32 [..., N, d], LSE [..., N].

    The arithmetic the merge kernel implements, written with tensor operations (the CPU steps use it).
    """
    o_part = o_part.float()
    if o_acc is None:
        return o_part, lse_part.clone()
    lse_new = torch.logaddexp(lse_acc, lse_part)
    # rows that saw no key in either part keep -inf / zero
    w_acc = torch.exp(lse_acc - lse_new).nan_to_num(nan=0.0).unsqueeze(-1)
    w_part = torch.exp(lse_part - lse_new).nan_to_num(nan=0.0).unsqueeze(-1)
    return o_acc * w_acc + o_part * w_part, lse_new


class KernelSteps:
    """The compute steps of a ring pass on a GPU: the library's kernels, nothing else."""

    def __init__(self):
        import flash_attn_legacy_cuda as ext
        self.ext = ext

    def fwd(self, q, k, v, scale, causal):
        """-> (O fp16, LSE fp32) of the queries over this key shard."""
        return self.ext.forward_rect(q, k, v, scale, causal)

    def merge(self, o_acc, lse_acc, o_part, lse_part, init):
        """(o_acc fp32, lse_acc) <- merged with the partial, in place (`init`: accumulators are empty)."""
        self.ext.merge_partial(o_acc, lse_acc, o_part, lse_part, init)

    def bwd(self, d_out, q, k, v, o, lse, scale, causal, dq_acc, dk_part, dv_part):
        """dq_acc += this pair's dQ before the softmax scale; dk_part / dv_part <- this pair's dK, dV (fp32)."""
        self.ext.backward_partial(d_out, q, k, v, o, lse, scale, causal, dq_acc, dk_part, dv_part)

    def add(self, dst, src):
        """dst += src (fp32)."""
        self.ext.accumulate_f32(dst, src)

    def cast(self, src, scale, dtype):
        """scale * src rounded to the model dtype: the one rounding of a gradient."""
        out = self.ext.scale_cast_f16(src, scale)
        return out if dtype == torch.float16 else out.to(dtype)


def _exchange(send: List[torch.Tensor], recv: List[torch.Tensor], group, rank: int, world: int):
    """Posts the sends to the next rank and the receives from the previous one; returns requests."""
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    ops = []
    for t in send:
        ops.append(dist.P2POp(dist.isend, t, dist.get_global_rank(group, nxt) if group else nxt, group))
    for t in recv:
        ops.append(dist.P2POp(dist.irecv, t, dist.get_global_rank(group, prv) if group else prv, group))
    return dist.batch_isend_irecv(ops)


def _wait_all(reqs, timeout_s: Optional[float], on_host: bool):
    """Waits for posted transfers.  With a time limit and host-side completion (CPU tensors) the
    backend's timed wait is used and its expiry becomes RingTimeoutError; otherwise it is the
    backend's plain wait (for CUDA tensors a stream dependency that does not block the host)."""
    if timeout_s is None or not on_host:
        for r in reqs:
            r.wait()
        return
    deadline = time.monotonic() + timeout_s
    for r in reqs:
        left = max(deadline - time.monotonic(), 0.001)
        try:
            r.wait(timeout=datetime.timedelta(seconds=left))
        except RuntimeError as e:
            if "imed out" in str(e):
                raise RingTimeoutError(f"a ring neighbour's shard did not arrive within {timeout_s} s") from e
            raise


class _ShardRing:
    """The K/V (or any) shards a rank holds while they travel the ring.

    `cur` starts as the caller's own tensors, which are only ever sent; shards received later
    land alternately in two private buffers, so the caller's tensors are never written.
    """

    def __init__(self, tensors, group, rank: int, world: int, timeout_s: Optional[float] = None):
        self.cur = [t.contiguous() for t in tensors]
        self._bufs = [None, None]
        self._turn = 0
        self._group, self._rank, self._world = group, rank, world
        self._incoming = None
        self._timeout_s = timeout_s
        self._on_host = not self.cur[0].is_cuda

    def start(self):
        """Posts send of `cur` to the next rank and receive of the previous rank's shards."""
        if self._bufs[self._turn] is None:
            self._bufs[self._turn] = [torch.empty_like(t) for t in self.cur]
        self._incoming = self._bufs[self._turn]
        return _exchange(self.cur, self._incoming, self._group, self._rank, self._world)

    def finish(self, reqs):
        """Waits for the posted exchange and makes the received shards current."""
        _wait_all(reqs, self._timeout_s, self._on_host)
        if self._incoming is not None:
            self.cur = self._incoming
            self._incoming = None
            self._turn ^= 1


def check_ring_shards(tensors, group=None):
    """Raises RingShardError on EVERY rank unless all ranks hold the same shapes and dtypes.

    One small all-gather of the shape descriptors, before any shard moves: a rank that was handed a
    shard of another length would otherwise receive into buffers of the wrong size (an error on one
    rank, a hang on its neighbours).
    """
    world = dist.get_world_size(group)
    desc = []
    for t in tensors:
        desc += [t.dim(), int(t.element_size()), int(t.is_floating_point())] + list(t.shape)
    mine = torch.tensor([len(desc)] + desc + [0] * (63 - len(desc)), dtype=torch.int64, device=tensors[0].device)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine, group=group)
    rows = [e.cpu().tolist() for e in everyone]
    if any(r != rows[0] for r in rows):
        bad = [i for i, r in enumerate(rows) if r != rows[0]]
        raise RingShardError(f"ring shards differ between ranks: ranks {bad} do not match rank 0")


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
                           steps=None, layout: str = "contiguous", timeout_s: Optional[float] = None,
                           check_shards: bool = True):
    """Forward over a sequence sharded across the ranks of `group`.

    q [B,Hq,Nl,d], k/v [B,Hkv,Nl,d]: this rank's rows (contiguous shard, or its two zigzag chunks
    back to back).  Returns (O [B,Hq,Nl,d] in q's dtype, LSE fp32 [B,Hq,Nl]) for this rank's
    rows, equal to attention over the whole sequence.  The inputs are not modified.
    `steps`: the compute steps (default: the library's kernels).  `timeout_s`: see the module text.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    zigzag = _check_layout(layout, causal, q.shape[2])
    if check_shards:
        check_ring_shards([q, k, v], group)
    if steps is None:
        steps = KernelSteps()
    rows = q.shape[2]
    kv = _ShardRing([k, v], group, rank, world, timeout_s)
    o_acc = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    lse_acc = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    for step in range(world):
        reqs = kv.start() if step + 1 < world else []
        plan = _shard_plan(zigzag, causal, rank, (rank - step) % world, rows)
        if plan is not None:
            qs, ks, masked = plan
            k_cur, v_cur = kv.cur
            o_p, lse_p = steps.fwd(q[:, :, qs], k_cur[:, :, ks], v_cur[:, :, ks], softmax_scale, masked)
            # step 0 is the diagonal and covers every local row: it initialises the accumulators
            steps.merge(o_acc[:, :, qs], lse_acc[:, :, qs], o_p, lse_p, step == 0)
        kv.finish(reqs)
    return steps.cast(o_acc, 1.0, q.dtype), lse_acc


def ring_attention_backward(d_out, q, k, v, o, lse, softmax_scale: float, causal: bool = True, group=None,
                            steps=None, layout: str = "contiguous", timeout_s: Optional[float] = None,
                            check_shards: bool = True):
    """Backward of `ring_attention_forward`.  `o`, `lse` are its outputs for this rank's rows.

    dQ stays local: the kernels add every shard pair's contribution into one fp32 accumulator.
    Each K/V shard travels the ring together with its fp32 dK/dV accumulator, which takes each
    rank's unrounded partial; after the last step one more hop returns the accumulator to the
    shard's owner.  Returns (dQ, dK, dV) for this rank's rows.  The inputs are not modified.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    zigzag = _check_layout(layout, causal, q.shape[2])
    if check_shards:
        check_ring_shards([d_out, q, k, v, o, lse], group)
    if steps is None:
        steps = KernelSteps()
    rows = q.shape[2]
    kv = _ShardRing([k, v], group, rank, world, timeout_s)
    grads = _ShardRing([torch.zeros(k.shape, dtype=torch.float32, device=k.device),
                        torch.zeros(v.shape, dtype=torch.float32, device=v.device)], group, rank, world, timeout_s)
    dq_acc = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    dk_part = torch.empty(k.shape, dtype=torch.float32, device=k.device)
    dv_part = torch.empty(v.shape, dtype=torch.float32, device=v.device)
    grads_in_flight = None
    for step in range(world):
        # K/V of the next step move while this step computes.  The gradient accumulators of the
        # shard held now were sent by the previous rank after ITS previous step: that transfer is
        # left in flight during this step's kernels and only waited for when their result is added.
        kv_reqs = kv.start() if step + 1 < world else []
        plan = _shard_plan(zigzag, causal, rank, (rank - step) % world, rows)
        if plan is not None:
            qs, ks, masked = plan
            k_cur, v_cur = kv.cur
            steps.bwd(d_out[:, :, qs], q[:, :, qs], k_cur[:, :, ks], v_cur[:, :, ks], o[:, :, qs],
                      lse[:, :, qs], softmax_scale, masked, dq_acc[:, :, qs], dk_part[:, :, ks], dv_part[:, :, ks])
        if grads_in_flight is not None:
            grads.finish(grads_in_flight)
        if plan is not None:
            dk_cur, dv_cur = grads.cur
            steps.add(dk_cur[:, :, ks], dk_part[:, :, ks])
            steps.add(dv_cur[:, :, ks], dv_part[:, :, ks])
        kv.finish(kv_reqs)
        grads_in_flight = grads.start()
    grads.finish(grads_in_flight)
    # After `world` hops every accumulator is back at its owner.
    dk_own, dv_own = grads.cur
    return (steps.cast(dq_acc, softmax_scale, q.dtype), steps.cast(dk_own, 1.0, k.dtype),
            steps.cast(dv_own, 1.0, v.dtype))
