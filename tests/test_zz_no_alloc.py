"""GPU: the allocation-free decode entry point (fal_decode_static) against fal_decode.

Who needs it: callers that cannot allocate device memory where they decode -- a serving loop
living inside a memory budget fixed at start-up, an operator callback that is handed only the
operator's own tensors, code that must avoid the device synchronisation an allocation can
trigger.  For them the split-K partials sit in an 8 MiB array inside the library instead of a
caller-provided workspace.  The results must be those of the regular entry point, call after
call, whatever an earlier call left in the shared array.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math
import os
import subprocess
import sys

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    import flash_attn_legacy_cuda as m
    return m


def _case(seed, B, Hq, Hkv, S, d, lens, append):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *shape: torch.randn(*shape, generator=g).half().cuda()
    kc, vc, q = mk(B, S, Hkv, d), mk(B, S, Hkv, d), mk(B, Hq, d)
    kn, vn = (mk(B, Hkv, d), mk(B, Hkv, d)) if append else (None, None)
    return q, kc, vc, torch.tensor(lens, dtype=torch.int32).cuda(), kn, vn


def test_static_decode_matches_regular_decode_on_two_calls_in_a_row(ext):
    # Two different problems back to back: the second call finds the first call's partials in the
    # shared array (a longer sequence layout first, a shorter one second) and must not be affected.
    cases = [
        _case(1, 4, 32, 8, 6000, 128, [6000, 1, 2049, 1024], append=False),
        _case(2, 3, 8, 2, 3000, 64, [17, 2999, 0], append=True),
    ]
    for q, kc, vc, lens, kn, vn in cases:
        B, Hq, d = q.shape
        scale = 1 / math.sqrt(d)
        kc2, vc2 = kc.clone(), vc.clone()
        o_ref, lse_ref = ext.decode(q, kc, vc, lens, scale, kn, vn, return_lse=True)
        out = torch.empty(B, Hq, d, dtype=torch.float16, device="cuda")
        lse = torch.empty(B, Hq, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        ext.decode_static(q, kc2, vc2, lens, scale, out, kn, vn, lse=lse)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before      # the binding allocated nothing either
        # same kernels, same inputs: the results are identical, well inside the parity tolerance
        assert (out.float() - o_ref.float()).abs().max().item() <= 2e-3 * o_ref.float().abs().max().item()
        assert (lse - lse_ref).abs().max().item() <= 1e-3
        assert torch.equal(out, o_ref)
        assert torch.equal(kc2, kc) and torch.equal(vc2, vc)   # the append wrote the same rows
        # and against the CPU oracle, so that this file stands on its own
        seen = lens.cpu() + (1 if kn is not None else 0)
        o_orc, lse_orc = orc.decode_fwd(q.cpu(), kc2.cpu(), vc2.cpu(), seen, scale)
        assert orc.rel_max_err(out, o_orc) <= orc.TOL_O and orc.abs_max_err(lse, lse_orc) <= orc.TOL_LSE
    assert ext.device_status() == 0


_FRESH_PROCESS = r"""
import math, torch
import flash_attn_legacy_cuda as ext
g = torch.Generator().manual_seed(5)
B, Hq, Hkv, S, d = 2, 8, 2, 1500, 128
mk = lambda *shape: torch.randn(*shape, generator=g).half().cuda()
q, kc, vc, kn, vn = mk(B, Hq, d), mk(B, S, Hkv, d), mk(B, S, Hkv, d), mk(B, Hkv, d), mk(B, Hkv, d)
lens = torch.tensor([1499, 3], dtype=torch.int32).cuda()
out = torch.empty(B, Hq, d, dtype=torch.float16, device="cuda")
lse = torch.empty(B, Hq, dtype=torch.float32, device="cuda")
ext.reset_device_status()          # start-up: creates the 4-byte status word, the module's only allocation
torch.cuda.synchronize()
before, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
ext.decode_static(q, kc, vc, lens, 1 / math.sqrt(d), out, kn, vn, lse=lse)   # the FIRST call in this process
torch.cuda.synchronize()
assert torch.cuda.memory_allocated() == before and torch.cuda.memory_reserved() == reserved
ref = ext.decode(q, kc.clone(), vc.clone(), lens + 1, 1 / math.sqrt(d))
assert torch.equal(out, ref)
assert ext.device_status() == 0
print("FRESH-OK")
"""


def test_first_static_call_of_a_process_allocates_nothing():
    """In a process of its own, so that no earlier call has warmed anything up: after the status word
    exists, the very first decode_static call leaves torch's allocator untouched."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(root, "flash-attention-legacy_b200"), root,
                                                       os.environ.get("PYTHONPATH", "")]))
    res = subprocess.run([sys.executable, "-c", _FRESH_PROCESS], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "FRESH-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_static_decode_rejects_problems_beyond_its_scratch(ext):
    # batch 64 x 32 heads x 32 splits x 130 floats = 34 MB of partials: beyond the 8 MiB array.
    lib = ctypes.CDLL(ext.LIB_PATH)
    lib.fal_decode_workspace_bytes.restype = ctypes.c_size_t
    assert lib.fal_decode_workspace_bytes(64, 32, 32768, 128) > ext.DECODE_STATIC_SCRATCH_BYTES
    q = torch.zeros(64, 32, 128, dtype=torch.float16, device="cuda")
    # a tiny cache view with a large logical capacity is enough: validation fails before any launch
    kc = torch.zeros(64, 1, 8, 128, dtype=torch.float16, device="cuda").expand(64, 32768, 8, 128)
    lens = torch.ones(64, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="fixed 8 MiB scratch"):
        ext.decode_static(q, kc, kc, lens, 0.1, torch.empty_like(q))
    assert ext.device_status() == 0
