"""GPU (2 or more devices): ring / context-parallel attention with the library's kernels as the
compute steps and NCCL point-to-point for the K/V exchange, against the single-GPU kernels and
the CPU oracle.  Skipped on a one-GPU machine."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results, layout):
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
        from oracle import attention_oracle as orc

        B, Hq, Hkv, N, d = 1, 8, 2, 1024 * world, 128
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
        o_ref, lse_ref = orc.attention_fwd_blocked(q, k, v, scale, True)
        dq_ref, dk_ref, dv_ref = orc.attention_bwd_blocked(q, k, v, do, scale, True)
        results[rank] = [orc.rel_max_err(o, take(o_ref)), orc.abs_max_err(lse, take(lse_ref)),
                         orc.rel_max_err(dq, take(dq_ref)), orc.rel_max_err(dk, take(dk_ref)),
                         orc.rel_max_err(dv, take(dv_ref)), ext.device_status()]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_ring_attention_on_gpus(layout):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results, layout), nprocs=world, join=True)
    assert len(results) == world
    for rank, (eo, el, edq, edk, edv, status) in results.items():
        assert eo <= 2e-3 and el <= 1e-3, (rank, eo, el)
        assert max(edq, edk, edv) <= 1e-2, (rank, edq, edk, edv)
        assert status == 0
