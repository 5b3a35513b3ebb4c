"""GPU: what the kernels do when something cannot complete -- without faulting, trapping or hanging
the device.  (The host-side cases -- a rank that stops between ring steps, a shard of the wrong size --
are in test_distributed_cpu.py.)"""
import math
import time

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ext():
    import flash_attn_legacy_cuda as m
    m.reset_device_status()
    yield m
    m.reset_device_status()


def test_a_wait_that_cannot_complete_ends_with_an_error_code(ext):
    """The library's self-test block waits on a barrier nobody arrives on, through the wait routine and
    the time limit (about a second) of the attention kernels.  It must come back by itself, leave
    1000 + barrier id in the status word, and the device must run the next kernel normally."""
    t0 = time.monotonic()
    status, gave_up = ext.selftest_wait_timeout(barrier_id=7)
    seconds = time.monotonic() - t0
    assert status == 1007
    assert gave_up == 2              # both warps of the block gave up; none is still spinning
    assert 0.2 < seconds < 10.0      # the limit is 2e9 cycles: about a second at the boost clock
    assert ext.device_status() == 1007   # sticky until it is reset
    ext.reset_device_status()
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 2, 200, 64, generator=g).half() for _ in range(3))
    o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), 0.125, True)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, 0.125, True)
    assert orc.rel_max_err(o, o_ref) <= orc.TOL_O and orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE
    assert ext.device_status() == 0


def test_a_token_that_does_not_fit_the_cache_is_reported_not_written(ext):
    """Decode with an append against a full cache: the entry attends to what is cached, nothing is
    written past the end, and the status word says that a token was dropped (2000)."""
    g = torch.Generator().manual_seed(2)
    B, S, hkv, hq, d = 3, 1024, 2, 8, 128
    kc, vc = torch.randn(B, S, hkv, d, generator=g).half(), torch.randn(B, S, hkv, d, generator=g).half()
    q, kn, vn = (torch.randn(B, h, d, generator=g).half() for h in (hq, hkv, hkv))
    lens = torch.tensor([S, 10, S - 1], dtype=torch.int32)      # entry 0 is full
    # the caches are views of larger buffers: rows written past the end would show up in the guard
    kbuf = torch.zeros(B, S + 8, hkv, d, dtype=torch.float16, device="cuda")
    vbuf = torch.zeros_like(kbuf)
    kbuf[:, :S], vbuf[:, :S] = kc.cuda(), vc.cuda()
    scale = 1 / math.sqrt(d)
    o, lse = ext.decode(q.cuda(), kbuf[:, :S], vbuf[:, :S], lens.cuda(), scale, kn.cuda(), vn.cuda(), return_lse=True)
    assert ext.device_status() == 2000
    assert (kbuf[:, S:] == 0).all() and (vbuf[:, S:] == 0).all()
    for b in (1, 2):
        kc[b, lens[b]] = kn[b]
        vc[b, lens[b]] = vn[b]
    assert torch.equal(kbuf[:, :S].cpu(), kc) and torch.equal(vbuf[:, :S].cpu(), vc)
    o_ref, lse_ref = orc.decode_fwd(q, kc, vc, torch.tensor([S, 11, S], dtype=torch.int32), scale)
    assert orc.rel_max_err(o, o_ref) <= orc.TOL_O and orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE


def test_binding_checks_every_buffer_a_decode_call_touches(ext):
    d, hq, hkv, B, S = 64, 8, 2, 2, 300
    q = torch.zeros(B, hq, d, dtype=torch.float16, device="cuda")
    kc = torch.zeros(B, S, hkv, d, dtype=torch.float16, device="cuda")
    lens = torch.ones(B, dtype=torch.int32, device="cuda")
    good_out = torch.empty(B, hq, d, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):   # out too small
        ext.decode(q, kc, kc, lens, 0.1, out=torch.empty(B, hq - 1, d, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):   # lengths for another batch size
        ext.decode(q, kc, kc, lens[:1], 0.1)
    with pytest.raises(RuntimeError):   # a new key of the wrong shape
        bad = torch.zeros(B, hkv + 1, d, dtype=torch.float16, device="cuda")
        ext.decode(q, kc, kc, lens, 0.1, bad, bad)
    with pytest.raises(RuntimeError):   # lse of the wrong dtype
        ext.decode_static(q, kc, kc, lens, 0.1, good_out, lse=torch.empty(B, hq, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):   # caches that disagree
        ext.decode_static(q, kc, kc[:, :10], lens, 0.1, good_out)
    assert ext.device_status() == 0
