"""CPU, gloo, world_size 2 to 4: the sharding helpers and the ring KV exchange.

The ring's compute steps are injected, so here they are the fp32 oracle; what is under test is the
exchange schedule, the causal shard skipping, the exact merge of partials, the travelling dK/dV
accumulators and the host-side failure detection (a rank that stops between steps, a shard of the
wrong size).  The same functions run on GPUs with the library's kernels as the compute steps.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_bwd(d_out, q, k, v, o, lse, scale, causal):
    # Gradient of THIS shard pair given the final statistics of the whole row: recompute P from
    # the global LSE, exactly what the kernels do.
    reps = q.shape[1] // k.shape[1]
    kf = k.float().repeat_interleave(reps, 1)
    vf = v.float().repeat_interleave(reps, 1)
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * scale
    if causal:
        n = s.shape[-1]
        s.masked_fill_(torch.triu(torch.ones(s.shape[-2], n, dtype=torch.bool), 1), float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    g = d_out.float()
    delta = (g * o.float()).sum(-1, keepdim=True)
    ds = p * (torch.matmul(g, vf.transpose(-1, -2)) - delta)
    b, hkv, nk, d = k.shape
    dq = torch.matmul(ds, kf) * scale
    dk = (torch.matmul(ds.transpose(-1, -2), q.float()) * scale).view(b, hkv, reps, nk, d).sum(2)
    dv = torch.matmul(p.transpose(-1, -2), g).view(b, hkv, reps, nk, d).sum(2)
    return dq, dk, dv


class OracleSteps:
    """The ring's compute steps on the CPU: the fp32 oracle and plain tensor arithmetic, with the
    contracts of flash_attn_legacy.distributed.KernelSteps."""

    def fwd(self, q, k, v, scale, causal):
        return orc.attention_fwd(q, k, v, scale, causal)

    def merge(self, o_acc, lse_acc, o_part, lse_part, init):
        import flash_attn_legacy.distributed as fd
        if init:
            o_acc.copy_(o_part)
            lse_acc.copy_(lse_part)
        else:
            o_new, lse_new = fd.merge_partials(o_acc.clone(), lse_acc.clone(), o_part, lse_part)
            o_acc.copy_(o_new)
            lse_acc.copy_(lse_new)

    def bwd(self, d_out, q, k, v, o, lse, scale, causal, dq_acc, dk_part, dv_part):
        dq, dk, dv = _oracle_bwd(d_out, q, k, v, o, lse, scale, causal)
        dq_acc += dq / scale          # the accumulator holds dQ before the softmax scale
        dk_part.copy_(dk)
        dv_part.copy_(dv)

    def add(self, dst, src):
        dst += src

    def cast(self, src, scale, dtype):
        return (src * scale).to(dtype)


def _ring_worker(rank, world, port, causal, results, layout="contiguous"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                        "flash-attention-legacy_b200"))
        from flash_attn_legacy import distributed as fd
        torch.manual_seed(0)
        B, Hq, Hkv, N, d = 1, 4, 2, 24 * world, 16
        q, k, v, g = torch.randn(B, Hq, N, d), torch.randn(B, Hkv, N, d), torch.randn(B, Hkv, N, d), torch.randn(B, Hq, N, d)
        if layout == "zigzag":
            def take(x):
                return fd.zigzag_take(x, world, rank)
        else:
            lo, hi = fd.shard_range(N, world, rank)

            def take(x):
                return x[:, :, lo:hi]
        # contiguous local tensors, reused by both calls: the exchange must leave them as they are
        ql, kl, vl, gl = (take(x).contiguous() for x in (q, k, v, g))
        o, lse = fd.ring_attention_forward(ql, kl, vl, 0.25, causal, None, OracleSteps(), layout)
        o_ref, lse_ref = orc.attention_fwd(q, k, v, 0.25, causal)
        dq, dk, dv = fd.ring_attention_backward(gl, ql, kl, vl, o, lse, 0.25, causal, None, OracleSteps(), layout)
        assert torch.equal(kl, take(k)) and torch.equal(vl, take(v)) and torch.equal(ql, take(q))
        dq_ref, dk_ref, dv_ref = orc.attention_bwd(q, k, v, g, 0.25, causal)
        errs = [(o - take(o_ref)).abs().max().item(), (lse - take(lse_ref)).abs().max().item(),
                (dq - take(dq_ref)).abs().max().item(), (dk - take(dk_ref)).abs().max().item(),
                (dv - take(dv_ref)).abs().max().item()]
        results[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("causal", [False, True])
def test_ring_attention_matches_full_attention(world, causal):
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_ring_worker, args=(world, port, causal, results), nprocs=world, join=True)
    assert len(results) == world
    for rank, errs in results.items():
        assert max(errs) < 1e-4, (rank, errs)


@pytest.mark.parametrize("world,causal", [(2, True), (4, True), (3, False)])
def test_zigzag_ring_attention_matches_full_attention(world, causal):
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_ring_worker, args=(world, port, causal, results, "zigzag"), nprocs=world, join=True)
    assert len(results) == world
    for rank, errs in results.items():
        assert max(errs) < 1e-4, (rank, errs)


def test_zigzag_rows_cover_the_sequence_once():
    import flash_attn_legacy.distributed as fd
    for world in (1, 2, 3, 4, 8):
        n = 2 * world * 5
        seen = []
        for r in range(world):
            (a0, a1), (b0, b1) = fd.zigzag_rows(n, world, r)
            assert a1 - a0 == b1 - b0 == 5 and a1 <= b0
            seen += list(range(a0, a1)) + list(range(b0, b1))
        assert sorted(seen) == list(range(n))
    with pytest.raises(ValueError):
        fd.zigzag_rows(10, 4, 0)


def test_shard_helpers():
    import flash_attn_legacy.distributed as fd
    # every unit assigned exactly once, sizes differ by at most one
    for n, w in ((32, 8), (16, 3), (5, 8), (64, 2)):
        spans = [fd.shard_range(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    # query heads follow their KV head: 32 query heads, 8 KV heads, 4 ranks
    qs, ks = fd.shard_heads(32, 8, 4, 1)
    assert (qs.start, qs.stop, ks.start, ks.stop) == (8, 16, 2, 4)


def test_merge_partials_is_exact():
    import flash_attn_legacy.distributed as fd
    torch.manual_seed(1)
    q, k, v = torch.randn(1, 2, 7, 8), torch.randn(1, 2, 20, 8), torch.randn(1, 2, 20, 8)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, 0.3, False)
    o1, l1 = orc.attention_fwd(q, k[:, :, :9], v[:, :, :9], 0.3, False)
    o2, l2 = orc.attention_fwd(q, k[:, :, 9:], v[:, :, 9:], 0.3, False)
    o, lse = fd.merge_partials(*fd.merge_partials(None, None, o1, l1), o2, l2)
    assert torch.allclose(o, o_ref, atol=1e-6) and torch.allclose(lse, lse_ref, atol=1e-6)
    # a part that saw no keys (LSE = -inf) leaves the other part unchanged
    o3, l3 = fd.merge_partials(o1, l1, torch.zeros_like(o1), torch.full_like(l1, float("-inf")))
    assert torch.allclose(o3, o1) and torch.allclose(l3, l1)


# ---------------------------------------------------------------------------------------------
# Failure detection on the host: no GPU is involved, nothing is made to fault
# ---------------------------------------------------------------------------------------------
class _LeavesAfterFirstStep(OracleSteps):
    """A rank that computes its first ring step and then stops taking part: it has posted the first
    exchange, it never posts the second."""

    class Left(Exception):
        pass

    def merge(self, o_acc, lse_acc, o_part, lse_part, init):
        super().merge(o_acc, lse_acc, o_part, lse_part, init)
        raise self.Left()


def _stalled_ring_worker(rank, world, port, results, release):
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                    "flash-attention-legacy_b200"))
    from flash_attn_legacy import distributed as fd
    torch.manual_seed(rank)
    q, k, v = torch.randn(1, 2, 8, 16), torch.randn(1, 2, 8, 16), torch.randn(1, 2, 8, 16)
    leaver = world - 1
    steps = _LeavesAfterFirstStep() if rank == leaver else OracleSteps()
    t0 = time.monotonic()
    try:
        fd.ring_attention_forward(q, k, v, 0.25, False, None, steps, "contiguous", timeout_s=2.0)
        outcome = "completed"
    except _LeavesAfterFirstStep.Left:
        outcome = "left"
    except fd.RingTimeoutError:
        outcome = "timeout"
    except RuntimeError as e:  # the transport itself noticed
        outcome = "transport error: " + str(e)[:80]
    results[rank] = (outcome, time.monotonic() - t0)
    # The rank that left stays alive (a stalled peer, not a dead one) until the others have reported.
    release.wait(timeout=60)
    os._exit(0)  # pending transfers to the stalled rank can never complete: skip the orderly shutdown


def test_a_rank_that_stops_between_ring_steps_is_detected_by_its_neighbours():
    """World 3, no mask (every rank has work in every step).  Rank 2 computes step 0 and stops.  Rank 0
    waits for the shard rank 2 should forward in step 1: it must give up with RingTimeoutError after the
    stated 2 s instead of blocking; rank 1 either finishes (it depends on rank 0 only) or reports too."""
    world = 3
    mgr = mp.Manager()
    results, release = mgr.dict(), mgr.Event()
    ctx = mp.spawn(_stalled_ring_worker, args=(world, _free_port(), results, release), nprocs=world, join=False)
    import time
    deadline = time.monotonic() + 40
    while len(results) < world and time.monotonic() < deadline:
        time.sleep(0.05)
    release.set()
    ctx.join(timeout=30)
    assert len(results) == world, dict(results)
    assert results[2][0] == "left"
    outcome0, seconds0 = results[0]
    assert outcome0 == "timeout" or outcome0.startswith("transport error"), dict(results)
    assert seconds0 < 10, seconds0
    assert results[1][0] in ("completed", "timeout") or results[1][0].startswith("transport error")
    assert results[1][1] < 20


def _wrong_shard_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                        "flash-attention-legacy_b200"))
        from flash_attn_legacy import distributed as fd

        class Counting(OracleSteps):
            calls = 0

            def fwd(self, *a):
                Counting.calls += 1
                return super().fwd(*a)

        rows = 8 if rank == 0 else 12  # rank 1 was handed a shard of another length
        q, k, v = torch.randn(1, 2, rows, 16), torch.randn(1, 2, rows, 16), torch.randn(1, 2, rows, 16)
        try:
            fd.ring_attention_forward(q, k, v, 0.25, True, None, Counting(), "contiguous")
            results[rank] = ("no error", Counting.calls)
        except fd.RingShardError:
            results[rank] = ("shard error", Counting.calls)
    finally:
        dist.destroy_process_group()


def test_a_shard_of_the_wrong_size_is_rejected_on_every_rank_before_anything_moves():
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_wrong_shard_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    assert dict(results) == {0: ("shard error", 0), 1: ("shard error", 0)}
