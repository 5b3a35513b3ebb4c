"""GPU: ring / context-parallel attention.

Two kinds of test.  (1) On ONE GPU the ring's arithmetic is run for every rank of a virtual ring in
turn: the same shard plan, the same step kernels (forward + merge, partial backward + fp32
accumulation, one final cast) as the multi-process code, with the transport replaced by indexing --
so the 8-rank numerics are pinned without 8 GPUs.  (2) On 2 or more GPUs the real thing: one process
per GPU, NCCL point-to-point for the K/V exchange, against the CPU oracle; skipped on a one-GPU
machine.
"""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ---------------------------------------------------------------------------------------------
# The step kernels on one GPU
# ---------------------------------------------------------------------------------------------
def test_merge_accumulate_and_cast_kernels():
    import flash_attn_legacy_cuda as ext
    from flash_attn_legacy import distributed as fd
    g = torch.Generator().manual_seed(3)
    B, H, N, d = 2, 3, 257, 128
    o_acc = torch.randn(B, H, N, d, generator=g)
    lse_acc = torch.randn(B, H, N, generator=g) * 3
    o_part = torch.randn(B, H, N, d, generator=g).half()
    lse_part = torch.randn(B, H, N, generator=g) * 3
    lse_acc[0, 0, :5] = float("-inf")     # rows the accumulator has not seen any key for
    lse_part[0, 1, :7] = float("-inf")    # rows this partial saw no key for
    lse_acc[1, 2, 3] = lse_part[1, 2, 3] = float("-inf")
    o_ref, lse_ref = fd.merge_partials(o_acc, lse_acc, o_part, lse_part)
    oa, la = o_acc.cuda(), lse_acc.cuda()
    ext.merge_partial(oa, la, o_part.cuda(), lse_part.cuda())
    assert torch.allclose(oa.cpu(), o_ref, atol=2e-6, rtol=1e-5)
    finite = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(la.cpu()), finite)
    assert (la.cpu()[finite] - lse_ref[finite]).abs().max().item() < 1e-5
    # a strided row range of larger accumulators, initialising them
    big_o = torch.full((B, H, 2 * N, d), float("nan"), device="cuda")
    big_l = torch.full((B, H, 2 * N), float("nan"), device="cuda")
    ext.merge_partial(big_o[:, :, N:], big_l[:, :, N:], o_part.cuda(), lse_part.cuda(), init=True)
    keep = torch.isfinite(lse_part).unsqueeze(-1)
    assert torch.equal(big_o[:, :, N:].cpu(), torch.where(keep, o_part.float(), torch.zeros(())))
    assert torch.equal(big_l[:, :, N:].cpu(), lse_part) and torch.isnan(big_o[:, :, :N]).all()

    a, b = torch.randn(B, H, N, 64, generator=g), torch.randn(B, H, 2 * N, 64, generator=g)
    ad, bd = a.cuda(), b.cuda()
    ext.accumulate_f32(ad, bd[:, :, :N])
    assert torch.equal(ad.cpu(), a + b[:, :, :N])
    assert torch.equal(ext.scale_cast_f16(ad, 0.125).cpu(), ((a + b[:, :, :N]) * 0.125).half())
    assert ext.device_status() == 0


def _virtual_ring(world, layout, q, k, v, do, scale):
    """Every rank of a `world`-rank causal ring, one after the other on this GPU: the shard plan and the
    step kernels of flash_attn_legacy.distributed, the exchange replaced by indexing.  Takes and
    returns full-sequence tensors (GPU)."""
    from flash_attn_legacy import distributed as fd
    steps = fd.KernelSteps()
    N = q.shape[2]

    def take(x, r):
        if layout == "zigzag":
            return fd.zigzag_take(x, world, r)
        lo, hi = fd.shard_range(N, world, r)
        return x[:, :, lo:hi].contiguous()

    local = [[take(t, r) for t in (q, k, v, do)] for r in range(world)]
    rows = local[0][0].shape[2]
    zig = layout == "zigzag"
    outs = []
    for r in range(world):
        ql, _, _, _ = local[r]
        o_acc = torch.empty(ql.shape, dtype=torch.float32, device="cuda")
        lse_acc = torch.empty(ql.shape[:3], dtype=torch.float32, device="cuda")
        for step in range(world):
            src = (r - step) % world
            plan = fd._shard_plan(zig, True, r, src, rows)
            if plan is None:
                continue
            qs, ks, masked = plan
            o_p, lse_p = steps.fwd(ql[:, :, qs], local[src][1][:, :, ks], local[src][2][:, :, ks], scale, masked)
            steps.merge(o_acc[:, :, qs], lse_acc[:, :, qs], o_p, lse_p, step == 0)
        outs.append((steps.cast(o_acc, 1.0, torch.float16), lse_acc))
    dk_acc = [torch.zeros(local[r][1].shape, dtype=torch.float32, device="cuda") for r in range(world)]
    dv_acc = [torch.zeros(local[r][2].shape, dtype=torch.float32, device="cuda") for r in range(world)]
    dqs = []
    for r in range(world):
        ql, _, _, dol = local[r]
        o, lse = outs[r]
        dq_acc = torch.zeros(ql.shape, dtype=torch.float32, device="cuda")
        dk_part = torch.empty(local[r][1].shape, dtype=torch.float32, device="cuda")
        dv_part = torch.empty_like(dk_part)
        for step in range(world):
            src = (r - step) % world
            plan = fd._shard_plan(zig, True, r, src, rows)
            if plan is None:
                continue
            qs, ks, masked = plan
            steps.bwd(dol[:, :, qs], ql[:, :, qs], local[src][1][:, :, ks], local[src][2][:, :, ks], o[:, :, qs],
                      lse[:, :, qs], scale, masked, dq_acc[:, :, qs], dk_part[:, :, ks], dv_part[:, :, ks])
            steps.add(dk_acc[src][:, :, ks], dk_part[:, :, ks])
            steps.add(dv_acc[src][:, :, ks], dv_part[:, :, ks])
        dqs.append(steps.cast(dq_acc, scale, torch.float16))

    def put(parts):
        full = torch.empty((parts[0].shape[0], parts[0].shape[1], N) + tuple(parts[0].shape[3:]),
                           dtype=parts[0].dtype, device="cuda")
        for r, part in enumerate(parts):
            if zig:
                (a0, a1), (b0, b1) = fd.zigzag_rows(N, world, r)
                full[:, :, a0:a1] = part[:, :, :a1 - a0]
                full[:, :, b0:b1] = part[:, :, a1 - a0:]
            else:
                lo, hi = fd.shard_range(N, world, r)
                full[:, :, lo:hi] = part
        return full

    return (put([x[0] for x in outs]), put([x[1] for x in outs]), put(dqs),
            put([steps.cast(t, 1.0, torch.float16) for t in dk_acc]),
            put([steps.cast(t, 1.0, torch.float16) for t in dv_acc]))


@pytest.mark.parametrize("world,layout", [(2, "contiguous"), (3, "contiguous"), (4, "zigzag"), (8, "zigzag")])
def test_ring_arithmetic_for_every_rank_on_one_gpu(world, layout):
    """512 rows per rank, GQA 4:1, checked in full against the oracle."""
    import flash_attn_legacy_cuda as ext
    B, Hq, Hkv, N, d = 1, 8, 2, 512 * world, 128
    g = torch.Generator().manual_seed(40 + world)
    q, k, v, do = (torch.randn(B, h, N, d, generator=g).half() for h in (Hq, Hkv, Hkv, Hq))
    scale = d ** -0.5
    o, lse, dq, dk, dv = _virtual_ring(world, layout, q.cuda(), k.cuda(), v.cuda(), do.cuda(), scale)
    o_ref, lse_ref = orc.attention_fwd_blocked(q, k, v, scale, True)
    assert orc.rel_max_err(o, o_ref) <= orc.TOL_O and orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE
    ref = orc.attention_bwd_blocked(q, k, v, do, scale, True)
    for name, got, want in zip(("dQ", "dK", "dV"), (dq, dk, dv), ref):
        assert orc.rel_max_err(got, want) <= orc.TOL_GRAD, name
    assert ext.device_status() == 0


def test_ring_arithmetic_at_eight_ranks_and_8192_rows_per_rank():
    """The long-context shape per rank (8 192 rows, zigzag, 8 ranks: N = 65 536) with one KV head and two
    query heads.  Gradients are summed in fp32 across the ring and rounded once, so the error must stay
    what a single-GPU backward has -- measured here on sampled row blocks (O, LSE, dQ), on the last 256
    keys (dK, dV) and against the single-GPU kernels on everything."""
    import flash_attn_legacy_cuda as ext
    B, Hq, Hkv, N, d, world = 1, 2, 1, 65536, 128, 8
    gen = torch.Generator(device="cuda").manual_seed(8)
    q = torch.randn(B, Hq, N, d, device="cuda", generator=gen).half()
    k = torch.randn(B, Hkv, N, d, device="cuda", generator=gen).half()
    v = torch.randn(B, Hkv, N, d, device="cuda", generator=gen).half()
    do = torch.randn(B, Hq, N, d, device="cuda", generator=gen).half()
    scale = d ** -0.5
    o, lse, dq, dk, dv = _virtual_ring(world, "zigzag", q, k, v, do, scale)
    assert ext.device_status() == 0
    kh, vh = k.cpu(), v.cpu()
    for r0 in (0, 8192 - 128, 40960, N - 256):   # a chunk boundary among them
        r1 = r0 + 256
        o_ref, lse_ref = orc.attention_fwd_rows(q[:, :, :r1].cpu(), kh, vh, scale, True, r0, r1)
        assert orc.rel_max_err(o[:, :, r0:r1], o_ref) <= orc.TOL_O
        assert orc.abs_max_err(lse[:, :, r0:r1], lse_ref) <= orc.TOL_LSE
        kf, vf = kh[:, :, :r1].float().expand(B, Hq, r1, d), vh[:, :, :r1].float().expand(B, Hq, r1, d)
        qf, gf = q[:, :, r0:r1].cpu().float(), do[:, :, r0:r1].cpu().float()
        s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        s.masked_fill_(torch.arange(r1).view(1, -1) > torch.arange(r0, r1).view(-1, 1), float("-inf"))
        p = torch.softmax(s, -1)
        ds = p * (torch.matmul(gf, vf.transpose(-1, -2)) - (gf * torch.matmul(p, vf)).sum(-1, keepdim=True))
        assert orc.rel_max_err(dq[:, :, r0:r1], torch.matmul(ds, kf) * scale) <= orc.TOL_GRAD
        if r1 == N:
            dk_ref = (torch.matmul(ds[..., r0:r1].transpose(-1, -2), qf) * scale).sum(1, keepdim=True)
            dv_ref = torch.matmul(p[..., r0:r1].transpose(-1, -2), gf).sum(1, keepdim=True)
            assert orc.rel_max_err(dk[:, :, r0:r1], dk_ref) <= orc.TOL_GRAD
            assert orc.rel_max_err(dv[:, :, r0:r1], dv_ref) <= orc.TOL_GRAD
    # everything against one single-GPU call (itself oracle-checked at this length by the long-context
    # test): the ring may differ from it by rounding only
    o1, lse1 = ext.forward(q, k, v, scale, True)
    g1 = ext.backward(do, q, k, v, o1, lse1, scale, True)
    assert orc.rel_max_err(o, o1.float().cpu()) <= orc.TOL_O
    assert orc.abs_max_err(lse, lse1.cpu()) <= orc.TOL_LSE
    for got, want in zip((dq, dk, dv), g1):
        assert orc.rel_max_err(got, want.float().cpu()) <= 2e-3   # a fifth of the gradient tolerance


# ---------------------------------------------------------------------------------------------
# The real ring: one process per GPU, NCCL
# ---------------------------------------------------------------------------------------------
def _worker(rank, world, port, results, layout, rows_per_rank):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sys
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        sys.path.insert(0, os.path.join(root, "flash-attention-legacy_b200"))
        sys.path.insert(0, root)
        from flash_attn_legacy import distributed as fd
        import flash_attn_legacy_cuda as ext

        full = rows_per_rank <= 1024
        B, Hq, Hkv, N, d = (1, 8, 2, rows_per_rank * world, 128) if full else (1, 2, 1, rows_per_rank * world, 128)
        g = torch.Generator().manual_seed(4)
        q, k, v, do = (torch.randn(B, h, N, d, generator=g).half() for h in (Hq, Hkv, Hkv, Hq))
        if layout == "zigzag":
            def take(x):
                return fd.zigzag_take(x, world, rank)
        else:
            lo, hi = fd.shard_range(N, world, rank)

            def take(x):
                return x[:, :, lo:hi]
        scale = d ** -0.5
        ql, kl, vl, dol = (take(t).contiguous().cuda() for t in (q, k, v, do))
        o, lse = fd.ring_attention_forward(ql, kl, vl, scale, True, layout=layout)
        dq, dk, dv = fd.ring_attention_backward(dol, ql, kl, vl, o, lse, scale, True, layout=layout)
        torch.cuda.synchronize()
        if full:
            o_ref, lse_ref = orc.attention_fwd_blocked(q, k, v, scale, True)
            dq_ref, dk_ref, dv_ref = orc.attention_bwd_blocked(q, k, v, do, scale, True)
            results[rank] = [orc.rel_max_err(o, take(o_ref)), orc.abs_max_err(lse, take(lse_ref)),
                             orc.rel_max_err(dq, take(dq_ref)), orc.rel_max_err(dk, take(dk_ref)),
                             orc.rel_max_err(dv, take(dv_ref)), ext.device_status()]
        else:
            # long shards: the single-GPU kernels on the whole sequence are the comparison (they are
            # checked against the oracle at this length by the one-GPU tests of this file)
            qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
            o1, lse1 = ext.forward(qc, kc, vc, scale, True)
            g1 = ext.backward(doc, qc, kc, vc, o1, lse1, scale, True)
            results[rank] = [orc.rel_max_err(o, take(o1).float().cpu()), orc.abs_max_err(lse, take(lse1).cpu()),
                             orc.rel_max_err(dq, take(g1[0]).float().cpu()),
                             orc.rel_max_err(dk, take(g1[1]).float().cpu()),
                             orc.rel_max_err(dv, take(g1[2]).float().cpu()), ext.device_status()]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout,rows_per_rank", [("contiguous", 1024), ("zigzag", 1024), ("zigzag", 8192)])
def test_ring_attention_on_gpus(layout, rows_per_rank):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results, layout, rows_per_rank), nprocs=world, join=True)
    assert len(results) == world
    for rank, (eo, el, edq, edk, edv, status) in results.items():
        assert eo <= 2e-3 and el <= 1e-3, (rank, eo, el)
        assert max(edq, edk, edv) <= 1e-2, (rank, edq, edk, edv)
        assert status == 0
