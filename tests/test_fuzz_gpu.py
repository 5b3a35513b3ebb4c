"""GPU: seeded random shapes through every entry of the binding against the CPU oracle.

The shapes are drawn around the tile edges (63..65, 127..129, 255..257, 511..513 rows), with GQA ratios
1, 2 and 4, all three head dims, empty sequences in packed batches and ragged cache lengths.  Gradients
are compared relative to max(|reference|, 0.5): with a handful of keys or a saturated softmax the true
gradient is nearly zero and only the absolute error of the fp16 P / dS rounding (which the reference
kernels share) is left, which a purely relative measure would blow up.
"""
import math
import random

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

EDGE_ROWS = [1, 2, 3, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 511, 512, 513, 700, 1025]


@pytest.fixture(scope="module")
def ext():
    import flash_attn_legacy_cuda as m
    m.reset_device_status()
    return m


def _rnd(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).half()


def _grad_ok(got, ref):
    ref = ref.float()
    err = (got.float().cpu() - ref).abs().max().item()
    return err <= orc.TOL_GRAD * max(ref.abs().max().item(), 0.5)


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes(ext, seed):
    rng = random.Random(1000 + seed)
    for _ in range(16):
        gen = torch.Generator().manual_seed(rng.randrange(1 << 30))
        kind = rng.choice(["batched", "batched", "varlen", "decode", "rect"])
        d = rng.choice([64, 128, 128, 256]) if kind != "rect" else rng.choice([64, 128])
        hkv = rng.choice([1, 2, 3])
        hq = hkv * rng.choice([1, 2, 4])
        causal = rng.random() < 0.6
        scale = rng.choice([1 / math.sqrt(d), 0.05])
        mag = rng.choice([1.0, 2.0])
        if kind == "batched":
            b, n = rng.choice([1, 2]), rng.choice(EDGE_ROWS)
            q, k = _rnd(gen, b, hq, n, d, scale=mag), _rnd(gen, b, hkv, n, d, scale=mag)
            v, do = _rnd(gen, b, hkv, n, d), _rnd(gen, b, hq, n, d)
            what = f"batched b{b} hq{hq} hkv{hkv} n{n} d{d} causal={causal} scale={scale:.3f} mag={mag}"
            o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), scale, causal)
            o_ref, lse_ref = orc.attention_fwd(q, k, v, scale, causal)
            assert orc.rel_max_err(o, o_ref) <= orc.TOL_O, what
            assert orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE, what
            grads = ext.backward(do.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, scale, causal)
            for g, r in zip(grads, orc.attention_bwd(q, k, v, do, scale, causal)):
                assert _grad_ok(g, r), what
        elif kind == "rect":
            nq, nk = rng.choice([1, 100, 128, 300]), rng.choice([1, 64, 129, 400, 777])
            q, k, v = _rnd(gen, 1, hq, nq, d), _rnd(gen, 1, hkv, nk, d), _rnd(gen, 1, hkv, nk, d)
            what = f"rect hq{hq} hkv{hkv} nq{nq} nk{nk} d{d}"
            o, lse = ext.forward_rect(q.cuda(), k.cuda(), v.cuda(), scale, False)
            o_ref, lse_ref = orc.attention_fwd(q, k, v, scale, False)
            assert orc.rel_max_err(o, o_ref) <= orc.TOL_O, what
            assert orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE, what
        elif kind == "varlen":
            lens = [rng.choice([0, 1, 5, 64, 127, 128, 129, 256, 300, 513, 600]) for _ in range(rng.choice([1, 2, 5, 9]))]
            if sum(lens) == 0:
                lens[0] = 7
            total = sum(lens)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
            q, k = _rnd(gen, total, hq, d, scale=mag), _rnd(gen, total, hkv, d, scale=mag)
            v, do = _rnd(gen, total, hkv, d), _rnd(gen, total, hq, d)
            what = f"varlen lens={lens} hq{hq} hkv{hkv} d{d} causal={causal} scale={scale:.3f} mag={mag}"
            o, lse = ext.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                        scale, causal)
            o_ref, lse_ref = orc.varlen_fwd(q, k, v, cu, cu, scale, causal)
            assert orc.rel_max_err(o, o_ref) <= orc.TOL_O, what
            assert orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE, what
            grads = ext.backward_varlen(do.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, cu.cuda(), cu.cuda(),
                                        max(lens), max(lens), scale, causal)
            for g, r in zip(grads, orc.varlen_bwd(q, k, v, do, cu, cu, scale, causal)):
                assert _grad_ok(g, r), what
        else:
            b, cap = rng.choice([1, 3]), rng.choice([64, 1000, 2048, 3000])
            kc, vc, qd = _rnd(gen, b, cap, hkv, d), _rnd(gen, b, cap, hkv, d), _rnd(gen, b, hq, d)
            seqlens = torch.tensor([rng.randint(1, cap) for _ in range(b)], dtype=torch.int32)
            what = f"decode b{b} hq{hq} hkv{hkv} cap{cap} d{d} lens={seqlens.tolist()}"
            out = ext.decode(qd.cuda(), kc.cuda(), vc.cuda(), seqlens.cuda(), scale)
            ref, _ = orc.decode_fwd(qd, kc, vc, seqlens, scale)
            assert orc.rel_max_err(out, ref) <= orc.TOL_O, what
        torch.cuda.synchronize()
        assert ext.device_status() == 0, what
