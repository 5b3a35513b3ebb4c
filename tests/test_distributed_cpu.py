"""CPU, gloo, world_size 2 and 3: the sharding helpers and the ring KV exchange.

The ring's compute steps are injected, so here they are the fp32 oracle; what is under test is the
exchange schedule, the causal shard skipping, the exact merge of partials and the travelling dK/dV
accumulators.  The same functions run on GPUs with the library's kernels as the compute steps.
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


def _oracle_fwd(q, k, v, scale, causal):
    return orc.attention_fwd(q, k, v, scale, causal)


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
        o, lse = fd.ring_attention_forward(ql, kl, vl, 0.25, causal, None, _oracle_fwd, layout)
        o_ref, lse_ref = orc.attention_fwd(q, k, v, 0.25, causal)
        dq, dk, dv = fd.ring_attention_backward(gl, ql, kl, vl, o, lse, 0.25, causal, None, _oracle_bwd, layout)
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
