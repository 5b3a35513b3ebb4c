"""GPU parity: the sm_100a kernels, called through the C-ABI binding, against the CPU oracle.

Tolerances (written once in oracle/attention_oracle.py):
    max|O - O_ref| / max|O_ref|  <= 2e-3,   same ratio <= 1e-2 for dQ, dK, dV,   max|LSE - LSE_ref| <= 1e-3.
The oracle consumes the same fp16 input bits as the kernels and computes in fp32.
"""
import math

import pytest
import torch

from conftest import golden_names, load_golden
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    import flash_attn_legacy_cuda as m
    m.reset_device_status()
    return m


@pytest.fixture(scope="module")
def fal():
    import flash_attn_legacy as m
    return m


def rand_half(gen, *shape):
    return torch.randn(*shape, generator=gen).half()


def check_fwd(o, lse, o_ref, lse_ref):
    assert orc.rel_max_err(o, o_ref) <= orc.TOL_O
    assert orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE


def check_grads(got, ref):
    for name, g, r in zip(("dQ", "dK", "dV"), got, ref):
        err = orc.rel_max_err(g, r)
        assert err <= orc.TOL_GRAD, f"{name}: {err}"


def run_fwd_bwd(ext, q, k, v, do, scale, causal):
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    o, lse = ext.forward(qc, kc, vc, scale, causal)
    grads = ext.backward(doc, qc, kc, vc, o, lse, scale, causal)
    return o, lse, grads


# ---------------------------------------------------------------------------------------------
# Golden vectors produced by the reference's own code
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", golden_names("batched_"))
def test_golden_batched(ext, name):
    g = load_golden(name)
    scale, causal = float(g["scale"]), bool(g["causal"])
    o, lse, grads = run_fwd_bwd(ext, g["q"], g["k"], g["v"], g["d_out"], scale, causal)
    assert orc.rel_max_err(o, g["o"]) <= orc.TOL_O
    check_grads(grads, (g["dq"], g["dk"], g["dv"]))
    _, lse_ref = orc.attention_fwd(g["q"], g["k"], g["v"], scale, causal)
    assert orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE


@pytest.mark.parametrize("name", golden_names("varlen_"))
def test_golden_varlen(ext, name):
    g = load_golden(name)
    cu = g["cu_seqlens"].cuda()
    lens = (g["cu_seqlens"][1:] - g["cu_seqlens"][:-1]).tolist()
    o, _ = ext.forward_varlen(g["q"].cuda(), g["k"].cuda(), g["v"].cuda(), cu, cu, max(lens), max(lens),
                              float(g["scale"]), bool(g["causal"]))
    assert orc.rel_max_err(o, g["o"]) <= orc.TOL_O


def test_golden_decode(ext):
    g = load_golden("decode_hook_d64")
    o = ext.decode(g["q"].cuda(), g["k_cache"].cuda(), g["v_cache"].cuda(), g["cache_seqlens"].cuda(),
                   float(g["scale"]))
    assert orc.rel_max_err(o, g["o"]) <= orc.TOL_O


# ---------------------------------------------------------------------------------------------
# Batched forward / backward against the oracle
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("n", [1, 33, 65, 100, 128, 200, 256, 257, 512, 777])
def test_forward_backward_shapes(ext, d, causal, n):
    g = torch.Generator().manual_seed(n * 7 + d)
    q, k, v, do = rand_half(g, 2, 4, n, d), rand_half(g, 2, 2, n, d), rand_half(g, 2, 2, n, d), rand_half(g, 2, 4, n, d)
    scale = 1 / math.sqrt(d)
    o, lse, grads = run_fwd_bwd(ext, q, k, v, do, scale, causal)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, scale, causal)
    check_fwd(o, lse, o_ref, lse_ref)
    ref = orc.attention_bwd(q, k, v, do, scale, causal)
    if n == 1:
        # dQ and dK are exactly zero for a single token; compare absolutely
        assert grads[0].abs().max().item() < 1e-3 and grads[1].abs().max().item() < 1e-3
        assert orc.rel_max_err(grads[2], ref[2]) <= orc.TOL_GRAD
    else:
        check_grads(grads, ref)
    assert ext.device_status() == 0


@pytest.mark.parametrize("hq,hkv", [(8, 2), (8, 4), (8, 1), (4, 1), (4, 2), (8, 8), (32, 1)])
def test_gqa_ratios(ext, hq, hkv):
    g = torch.Generator().manual_seed(hq * 10 + hkv)
    n, d = 160, 64
    q, k, v, do = rand_half(g, 1, hq, n, d), rand_half(g, 1, hkv, n, d), rand_half(g, 1, hkv, n, d), rand_half(g, 1, hq, n, d)
    o, lse, grads = run_fwd_bwd(ext, q, k, v, do, 0.125, True)
    check_fwd(o, lse, *orc.attention_fwd(q, k, v, 0.125, True))
    check_grads(grads, orc.attention_bwd(q, k, v, do, 0.125, True))
    assert grads[1].shape == k.shape and grads[2].shape == v.shape


def test_config1_mha_forward_n1024_d64(ext):
    """B=2, H=8, N=1024, d=64, causal, seed 0 -- checked in full."""
    g = torch.Generator().manual_seed(0)
    q, k, v = rand_half(g, 2, 8, 1024, 64), rand_half(g, 2, 8, 1024, 64), rand_half(g, 2, 8, 1024, 64)
    o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), 0.125, True)
    check_fwd(o, lse, *orc.attention_fwd(q, k, v, 0.125, True))


def test_config2_gqa_n4096_d128_full_size(ext):
    """B=4, Hq=32, Hkv=8, N=4096, d=128 causal forward + backward at full size on the GPU; the oracle
    checks 11 of the 32 (batch, kv-head) groups in full -- all eight of batch entry 0 and one of each
    other entry; the rest is covered by size-independent properties."""
    B, Hq, Hkv, N, d = 4, 32, 8, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(B, Hq, N, d, device="cuda", generator=gen).half()
    k = torch.randn(B, Hkv, N, d, device="cuda", generator=gen).half()
    v = torch.randn(B, Hkv, N, d, device="cuda", generator=gen).half()
    do = torch.randn(B, Hq, N, d, device="cuda", generator=gen).half()
    scale = 1 / math.sqrt(d)
    o, lse = ext.forward(q, k, v, scale, True)
    dq, dk, dv = ext.backward(do, q, k, v, o, lse, scale, True)
    for b, h in [(0, h) for h in range(8)] + [(1, 2), (2, 7), (3, 5)]:
        sl = slice(4 * h, 4 * h + 4)
        qs, ks, vs, gs = q[b:b + 1, sl].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu(), do[b:b + 1, sl].cpu()
        o_ref, lse_ref = orc.attention_fwd_blocked(qs, ks, vs, scale, True)
        check_fwd(o[b:b + 1, sl], lse[b:b + 1, sl], o_ref, lse_ref)
        ref = orc.attention_bwd_blocked(qs, ks, vs, gs, scale, True)
        check_grads((dq[b:b + 1, sl], dk[b:b + 1, h:h + 1], dv[b:b + 1, h:h + 1]), ref)
    # properties over the whole output: finite, causal first row equals V[0], a second run of the
    # forward is bitwise identical, and each batch entry computed alone gives the same forward bits.
    for t in (o, lse, dq, dk, dv):
        assert torch.isfinite(t).all()
    v_rep = v[:, :, 0].repeat_interleave(4, dim=1)
    assert (o[:, :, 0].float() - v_rep.float()).abs().max().item() < 2e-3
    o2, lse2 = ext.forward(q, k, v, scale, True)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    o_b, _ = ext.forward(q[2:3], k[2:3], v[2:3], scale, True)
    assert torch.equal(o_b, o[2:3])
    # dV is linear in dO: backward(2*dO).dV == 2*dV up to fp16 rounding of the doubled inputs
    _, _, dv2 = ext.backward(do * 2, q, k, v, o, lse, scale, True)
    assert orc.rel_max_err(dv2, dv.float().cpu() * 2) <= 2e-3
    assert ext.device_status() == 0


def test_forward_is_deterministic(ext):
    g = torch.Generator().manual_seed(5)
    q, k, v = (rand_half(g, 1, 4, 256, 128).cuda() for _ in range(3))
    a = ext.forward(q, k, v, 0.1, True)
    b = ext.forward(q, k, v, 0.1, True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_batch_independence(ext):
    g = torch.Generator().manual_seed(6)
    q, k, v = (rand_half(g, 4, 2, 128, 64).cuda() for _ in range(3))
    full, _ = ext.forward(q, k, v, 0.125, False)
    for b in range(4):
        one, _ = ext.forward(q[b:b + 1], k[b:b + 1], v[b:b + 1], 0.125, False)
        assert torch.equal(full[b:b + 1], one)


def test_zero_scores_give_mean_of_v(ext):
    g = torch.Generator().manual_seed(7)
    v = rand_half(g, 1, 1, 64, 64) * 0.1
    z = torch.zeros(1, 1, 64, 64, dtype=torch.float16)
    o, lse = ext.forward(z.cuda(), z.cuda(), v.cuda(), 0.125, False)
    expect = v.float().mean(dim=2, keepdim=True).expand_as(v)
    assert (o.float().cpu() - expect).abs().max().item() < 1e-3
    assert (lse.cpu() - math.log(64)).abs().max().item() < 1e-4


def test_large_magnitude_scores_stay_finite(ext):
    g = torch.Generator().manual_seed(8)
    q, k, v = rand_half(g, 1, 2, 300, 128) * 5, rand_half(g, 1, 2, 300, 128) * 5, rand_half(g, 1, 2, 300, 128)
    scale = 1 / math.sqrt(128)
    o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), scale, True)
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    check_fwd(o, lse, *orc.attention_fwd(q, k, v, scale, True))


def test_custom_scale(ext):
    g = torch.Generator().manual_seed(9)
    q, k, v = (rand_half(g, 1, 2, 96, 64) for _ in range(3))
    o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), 0.05, False)
    check_fwd(o, lse, *orc.attention_fwd(q, k, v, 0.05, False))


def test_strided_bnhd_inputs_without_copies(ext):
    """[B,N,H,d] storage viewed as [B,H,N,d] goes through the C-ABI strides unchanged."""
    g = torch.Generator().manual_seed(10)
    qs, ks, vs = rand_half(g, 2, 150, 4, 64), rand_half(g, 2, 150, 2, 64), rand_half(g, 2, 150, 2, 64)
    q, k, v = (t.cuda().transpose(1, 2) for t in (qs, ks, vs))
    assert not q.is_contiguous()
    o, lse = ext.forward(q, k, v, 0.125, True)
    check_fwd(o, lse, *orc.attention_fwd(qs.transpose(1, 2), ks.transpose(1, 2), vs.transpose(1, 2), 0.125, True))


def test_rectangular_forward_top_left_causal(ext):
    """seqlen_q != seqlen_k in the forward, causal mask aligned top-left as in the reference kernels."""
    g = torch.Generator().manual_seed(11)
    q, k, v = rand_half(g, 1, 2, 300, 64), rand_half(g, 1, 2, 170, 64), rand_half(g, 1, 2, 170, 64)
    for causal in (False, True):
        o, lse = ext.forward_rect(q.cuda(), k.cuda(), v.cuda(), 0.125, causal)
        check_fwd(o, lse, *orc.attention_fwd(q, k, v, 0.125, causal))


@pytest.mark.parametrize("tiles", [1, 2])
@pytest.mark.parametrize("d", [64, 128])
def test_every_forward_kernel_variant(ext, tiles, d):
    """Both forward variants -- one 128-row tile per thread block whose key tiles alternate between the
    two softmax warpgroups (1), two tiles with one warpgroup each (2) -- on the same problems; by
    default the library picks by grid size, so small problems would otherwise only ever see the first."""
    ext.set_forward_variant(tiles)
    try:
        for n, hq, hkv, causal in ((1, 4, 2, True), (100, 4, 2, True), (200, 2, 2, False), (257, 4, 4, False),
                                   (777, 8, 2, True),
                                   (1500, 4, 1, True), (2048, 2, 2, False)):
            g = torch.Generator().manual_seed(n + d + tiles)
            q, k, v = rand_half(g, 2, hq, n, d), rand_half(g, 2, hkv, n, d), rand_half(g, 2, hkv, n, d)
            scale = 1 / math.sqrt(d)
            o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), scale, causal)
            check_fwd(o, lse, *orc.attention_fwd(q, k, v, scale, causal))
            o2, lse2 = ext.forward(q.cuda(), k.cuda(), v.cuda(), scale, causal)
            assert torch.equal(o, o2) and torch.equal(lse, lse2)   # bitwise deterministic either way
        # large scores: the running maximum moves and O is rescaled (each column half its own columns)
        g = torch.Generator().manual_seed(77 + tiles)
        q, k, v = rand_half(g, 1, 2, 600, d) * 6, rand_half(g, 1, 2, 600, d) * 6, rand_half(g, 1, 2, 600, d)
        o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), 1 / math.sqrt(d), True)
        check_fwd(o, lse, *orc.attention_fwd(q, k, v, 1 / math.sqrt(d), True))
        # scores that keep growing along the keys: the maximum moves at most steps, so (variant 1) both
        # warpgroups rescale O and bring their private row sums onto the other's reference
        ramp = (1 + 7 * torch.arange(1500) / 1500).view(1, 1, 1500, 1)
        q, k, v = rand_half(g, 1, 2, 1500, d), (rand_half(g, 1, 2, 1500, d) * ramp).half(), rand_half(g, 1, 2, 1500, d)
        for causal in (False, True):
            o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), 1 / math.sqrt(d), causal)
            check_fwd(o, lse, *orc.attention_fwd(q, k, v, 1 / math.sqrt(d), causal))
        # packed sequences and the end-aligned mask
        lens = [300, 17, 1025, 256]
        qp, kp, vp, _, cu = packed_inputs(g, lens, 4, 2, d)
        o, lse = ext.forward_varlen(qp.cuda(), kp.cuda(), vp.cuda(), cu.cuda(), cu.cuda(), 1025, 1025, 0.1, True)
        check_fwd(o, lse, *orc.varlen_fwd(qp, kp, vp, cu, cu, 0.1, True))
        q, k, v = rand_half(g, 1, 4, 200, d), rand_half(g, 1, 2, 777, d), rand_half(g, 1, 2, 777, d)
        o, lse = ext.forward_rect(q.cuda(), k.cuda(), v.cuda(), 0.1, True, bottom_right=True)
        check_fwd(o, lse, *orc.attention_fwd(q, k, v, 0.1, True, causal_shift=577))
        assert ext.device_status() == 0
    finally:
        ext.set_forward_variant(0)


def test_seeded_sweep_of_small_shapes(ext):
    """Sixty seeded random problems -- lengths 1..700 with unequal query / key lengths, every head_dim,
    GQA ratios 1 / 2 / 4 / 8, no mask / the reference's mask / the end-aligned mask, both forward kernel
    variants as the library picks them -- forward and backward against the oracle."""
    rnd = torch.Generator().manual_seed(2024)
    pick = lambda choices: choices[int(torch.randint(len(choices), (1,), generator=rnd))]
    for case in range(60):
        d = pick([32, 64, 96, 128, 256])
        hkv = pick([1, 2, 3])
        hq = hkv * pick([1, 2, 4, 8])
        b = pick([1, 2, 3])
        nk = int(torch.randint(1, 701, (1,), generator=rnd))
        mode = pick([0, 1, 2])          # 0 no mask, 1 top-left causal, 2 end-aligned causal
        nq = nk if mode == 1 or pick([True, False]) else int(torch.randint(1, nk + 1, (1,), generator=rnd))
        scale = pick([1 / math.sqrt(d), 0.05, 0.3])
        q, k, v, do = (rand_half(rnd, b, hq, nq, d), rand_half(rnd, b, hkv, nk, d), rand_half(rnd, b, hkv, nk, d),
                       rand_half(rnd, b, hq, nq, d))
        shift = nk - nq if mode == 2 else 0
        where = f"case {case}: b{b} hq{hq} hkv{hkv} nq{nq} nk{nk} d{d} mode{mode}"
        o, lse = ext.forward_rect(q.cuda(), k.cuda(), v.cuda(), scale, mode != 0, bottom_right=mode == 2)
        o_ref, lse_ref = orc.attention_fwd(q, k, v, scale, mode != 0, causal_shift=shift)
        assert orc.rel_max_err(o, o_ref) <= orc.TOL_O, where
        assert orc.abs_max_err(lse, lse_ref) <= orc.TOL_LSE, where
        if nq == nk or mode == 2:       # the batched backward takes equal lengths or the end-aligned mask
            got = ext.backward(do.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, scale, mode != 0, bottom_right=mode == 2)
            ref = orc.attention_bwd(q, k, v, do, scale, mode != 0, causal_shift=shift)
            for g, r, name in zip(got, ref, ("dq", "dk", "dv")):
                assert orc.rel_max_err(g, r) <= orc.TOL_GRAD, f"{where} {name}"
    assert ext.device_status() == 0


# ---------------------------------------------------------------------------------------------
# Packed sequences
# ---------------------------------------------------------------------------------------------
def packed_inputs(gen, lens, h, hkv, d):
    total = sum(lens)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    return (rand_half(gen, total, h, d), rand_half(gen, total, hkv, d), rand_half(gen, total, hkv, d),
            rand_half(gen, total, h, d), cu)


@pytest.mark.parametrize("lens", [[32, 64, 48], [1, 1, 1, 1], [300, 17, 1025, 256, 511], [257], [64] * 9])
@pytest.mark.parametrize("d,h,hkv", [(64, 4, 4), (128, 8, 2)])
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_forward_backward(ext, lens, d, h, hkv, causal):
    g = torch.Generator().manual_seed(sum(lens) + d)
    q, k, v, do, cu = packed_inputs(g, lens, h, hkv, d)
    scale = 1 / math.sqrt(d)
    cuc = cu.cuda()
    o, lse = ext.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cuc, cuc, max(lens), max(lens), scale, causal)
    grads = ext.backward_varlen(do.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, cuc, cuc, max(lens), max(lens),
                                scale, causal)
    check_fwd(o, lse, *orc.varlen_fwd(q, k, v, cu, cu, scale, causal))
    ref = orc.varlen_bwd(q, k, v, do, cu, cu, scale, causal)
    if max(lens) == 1:
        assert grads[0].abs().max().item() < 1e-3 and grads[1].abs().max().item() < 1e-3
        assert orc.rel_max_err(grads[2], ref[2]) <= orc.TOL_GRAD
    else:
        check_grads(grads, ref)
    assert ext.device_status() == 0


def test_varlen_single_sequence_equals_batched(ext):
    g = torch.Generator().manual_seed(12)
    n, h, d = 200, 4, 64
    q, k, v = (rand_half(g, 1, h, n, d).cuda() for _ in range(3))
    ob, lb = ext.forward(q, k, v, 0.125, True)
    cu = torch.tensor([0, n], dtype=torch.int32).cuda()
    pk = lambda t: t[0].permute(1, 0, 2).contiguous()
    ov, lv = ext.forward_varlen(pk(q), pk(k), pk(v), cu, cu, n, n, 0.125, True)
    assert torch.equal(ov.permute(1, 0, 2), ob[0]) and torch.equal(lv.permute(1, 0), lb[0])


def test_varlen_unequal_q_and_k_lengths_forward(ext):
    g = torch.Generator().manual_seed(13)
    lq, lk = [40, 130, 7], [100, 60, 300]
    h, d = 2, 64
    cu_q = torch.tensor([0, 40, 170, 177], dtype=torch.int32)
    cu_k = torch.tensor([0, 100, 160, 460], dtype=torch.int32)
    q, k, v = rand_half(g, 177, h, d), rand_half(g, 460, h, d), rand_half(g, 460, h, d)
    for causal in (False, True):
        o, lse = ext.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), max(lq), max(lk),
                                    0.125, causal)
        check_fwd(o, lse, *orc.varlen_fwd(q, k, v, cu_q, cu_k, 0.125, causal))


def test_varlen_with_an_empty_sequence(ext):
    g = torch.Generator().manual_seed(14)
    lens = [50, 0, 90]
    q, k, v, do, cu = packed_inputs(g, lens, 2, 2, 64)
    o, lse = ext.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), 90, 90, 0.125, True)
    grads = ext.backward_varlen(do.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, cu.cuda(), cu.cuda(), 90, 90,
                                0.125, True)
    cu2 = torch.tensor([0, 50, 140], dtype=torch.int32)
    check_fwd(o, lse, *orc.varlen_fwd(q, k, v, cu2, cu2, 0.125, True))
    check_grads(grads, orc.varlen_bwd(q, k, v, do, cu2, cu2, 0.125, True))


def test_config3_varlen_16_sequences(ext):
    """16 sequences, lengths uniform in [64, 4096] (seed 2), H=16, d=128, causal, forward + backward at
    full size; the oracle checks four of the 16 heads on every sequence."""
    gl = torch.Generator().manual_seed(2)
    lens = torch.randint(64, 4097, (16,), generator=gl).tolist()
    total, H, d = sum(lens), 16, 128
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    gen = torch.Generator(device="cuda").manual_seed(2)
    q, k, v, do = (torch.randn(total, H, d, device="cuda", generator=gen).half() for _ in range(4))
    scale = 1 / math.sqrt(d)
    cuc = cu.cuda()
    o, lse = ext.forward_varlen(q, k, v, cuc, cuc, max(lens), max(lens), scale, True)
    dq, dk, dv = ext.backward_varlen(do, q, k, v, o, lse, cuc, cuc, max(lens), max(lens), scale, True)
    for t in (o, lse, dq, dk, dv):
        assert torch.isfinite(t).all()
    for h in (0, 5, 9, 15):
        sl = slice(h, h + 1)
        qs, ks, vs, gs = (t[:, sl].cpu() for t in (q, k, v, do))
        check_fwd(o[:, sl], lse[:, sl], *orc.varlen_fwd(qs, ks, vs, cu, cu, scale, True))
        check_grads((dq[:, sl], dk[:, sl], dv[:, sl]), orc.varlen_bwd(qs, ks, vs, gs, cu, cu, scale, True))
    # every sequence's first row sees only its own first key
    first = cu[:-1].long().cuda()
    assert (o[first].float() - v[first].float()).abs().max().item() < 2e-3
    assert ext.device_status() == 0


# ---------------------------------------------------------------------------------------------
# Decode
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 8), (64, 8, 8), (128, 8, 1), (64, 40, 2)])
@pytest.mark.parametrize("append", [False, True])
def test_decode_against_oracle(ext, d, hq, hkv, append):
    g = torch.Generator().manual_seed(d + hq + append)
    B, S = 5, 2500
    kc, vc = rand_half(g, B, S, hkv, d), rand_half(g, B, S, hkv, d)
    q = rand_half(g, B, hq, d)
    lens = torch.tensor([0 if append else 1, 15, 1024, 1025, 2499], dtype=torch.int32)
    kn, vn = (rand_half(g, B, hkv, d), rand_half(g, B, hkv, d)) if append else (None, None)
    kcc, vcc = kc.cuda(), vc.cuda()
    scale = 1 / math.sqrt(d)
    o, lse = ext.decode(q.cuda(), kcc, vcc, lens.cuda(), scale, kn.cuda() if append else None,
                        vn.cuda() if append else None, return_lse=True)
    if append:
        for b in range(B):
            kc[b, lens[b]] = kn[b]
            vc[b, lens[b]] = vn[b]
        assert torch.equal(kcc.cpu(), kc) and torch.equal(vcc.cpu(), vc)  # append wrote exactly one row each
        lens = lens + 1
    check_fwd(o, lse, *orc.decode_fwd(q, kc, vc, lens, scale))
    assert ext.device_status() == 0


def test_decode_hf_cache_layout(ext):
    g = torch.Generator().manual_seed(21)
    B, S, hkv, hq, d = 2, 700, 2, 8, 64
    kc, vc, q = rand_half(g, B, hkv, S, d), rand_half(g, B, hkv, S, d), rand_half(g, B, hq, d)
    lens = torch.tensor([700, 333], dtype=torch.int32)
    o = ext.decode(q.cuda(), kc.cuda(), vc.cuda(), lens.cuda(), 0.125, cache_layout="bhsd")
    o_ref, _ = orc.decode_fwd(q, kc.transpose(1, 2), vc.transpose(1, 2), lens, 0.125)
    assert orc.rel_max_err(o, o_ref) <= orc.TOL_O


@pytest.mark.parametrize("layout", ["bshd", "bhsd"])
def test_decode_skips_a_left_padded_prefix(ext, layout):
    """cache_starts: entry b attends to positions [start_b, len_b) (+ the appended one)."""
    g = torch.Generator().manual_seed(61)
    B, S, hkv, hq, d = 5, 2300, 2, 8, 128
    kc, vc, q = rand_half(g, B, S, hkv, d), rand_half(g, B, S, hkv, d), rand_half(g, B, hq, d)
    kn, vn = rand_half(g, B, hkv, d), rand_half(g, B, hkv, d)
    lens = torch.tensor([2299, 1500, 1024, 7, 2000], dtype=torch.int32)
    starts = torch.tensor([0, 1499, 1000, 7, 1025], dtype=torch.int32)   # entry 3: nothing but the new token
    kcc, vcc = kc.cuda(), vc.cuda()
    if layout == "bhsd":
        kcc, vcc = kcc.transpose(1, 2).contiguous(), vcc.transpose(1, 2).contiguous()
    o, lse = ext.decode(q.cuda(), kcc, vcc, lens.cuda(), 0.09, kn.cuda(), vn.cuda(), cache_layout=layout,
                        return_lse=True, cache_starts=starts.cuda())
    for b in range(B):
        kc[b, lens[b]] = kn[b]
        vc[b, lens[b]] = vn[b]
    check_fwd(o, lse, *orc.decode_fwd(q, kc, vc, lens + 1, 0.09, cache_starts=starts))
    # without an append, and an entry whose range is empty: zeros
    o2 = ext.decode(q.cuda(), kcc, vcc, lens.cuda(), 0.09, cache_layout=layout, cache_starts=starts.cuda())
    o2_ref, _ = orc.decode_fwd(q, kc, vc, lens, 0.09, cache_starts=starts)
    assert orc.rel_max_err(o2, o2_ref) <= orc.TOL_O and (o2[3] == 0).all()
    assert ext.device_status() == 0


def test_decode_step_replayed_as_a_cuda_graph(ext):
    """One decode step (append, split-K, combine, length increment) captured once and replayed: every
    replay must give what the oracle gives for the cache as it then stands.  (A small per-GPU batch is
    bound by the launch path; replaying a graph removes it.)"""
    g = torch.Generator().manual_seed(44)
    B, S, hkv, hq, d = 3, 2048, 2, 8, 128
    kc, vc = rand_half(g, B, S, hkv, d), rand_half(g, B, S, hkv, d)
    q, kn, vn = rand_half(g, B, hq, d), rand_half(g, B, hkv, d), rand_half(g, B, hkv, d)
    lens0 = torch.tensor([0, 1023, 2040], dtype=torch.int32)
    kc_d, vc_d, q_d, kn_d, vn_d = (t.cuda() for t in (kc, vc, q, kn, vn))
    lens = lens0.cuda()
    out = torch.empty(B, hq, d, dtype=torch.float16, device="cuda")
    scale = 1 / math.sqrt(d)
    scratch_k, scratch_v = kc_d.clone(), vc_d.clone()
    ext.decode(q_d, scratch_k, scratch_v, lens.clone(), scale, kn_d, vn_d, out=out)  # first call: one-time set-up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ext.decode(q_d, kc_d, vc_d, lens, scale, kn_d, vn_d, out=out)
        lens += 1
    lens.copy_(lens0.cuda())            # capture does not run the kernels; the caches are still untouched
    kc_ref, vc_ref = kc.clone(), vc.clone()
    for step in range(3):
        q_d.copy_(rand_half(g, B, hq, d))          # new inputs go into the captured buffers
        kn_d.copy_(rand_half(g, B, hkv, d))
        vn_d.copy_(rand_half(g, B, hkv, d))
        graph.replay()
        cur = lens0 + step
        for b in range(B):
            kc_ref[b, cur[b]] = kn_d[b].cpu()
            vc_ref[b, cur[b]] = vn_d[b].cpu()
        o_ref, _ = orc.decode_fwd(q_d.cpu(), kc_ref, vc_ref, cur + 1, scale)
        assert orc.rel_max_err(out, o_ref) <= orc.TOL_O, step
    assert lens.cpu().tolist() == (lens0 + 3).tolist()
    assert ext.device_status() == 0


def test_config4_decode_256_steps_with_appends(ext):
    """batch 64, Hq=32, Hkv=8, d=128, caches [64,32768,8,128], lengths uniform in [1024, 32768-256]
    (clamped so that 256 appended tokens fit), 256 decode steps with appends.  The oracle checks
    eight batch entries (the shortest and the longest among them) at steps 0, 64, 128, 192 and 255."""
    B, Hq, Hkv, S, d, steps = 64, 32, 8, 32768, 128, 256
    gen = torch.Generator(device="cuda").manual_seed(3)
    kc = torch.randn(B, S, Hkv, d, device="cuda", dtype=torch.float16, generator=gen)
    vc = torch.randn(B, S, Hkv, d, device="cuda", dtype=torch.float16, generator=gen)
    lens = torch.randint(1024, S - steps + 1, (B,), device="cuda", generator=gen).to(torch.int32)
    lens[0], lens[1] = 1024, S - steps
    scale = 1 / math.sqrt(d)
    picks = [0, 1, 9, 22, 37, 45, 58, 63]
    for step in range(steps):
        q = torch.randn(B, Hq, d, device="cuda", dtype=torch.float16, generator=gen)
        kn = torch.randn(B, Hkv, d, device="cuda", dtype=torch.float16, generator=gen)
        vn = torch.randn(B, Hkv, d, device="cuda", dtype=torch.float16, generator=gen)
        o, lse = ext.decode(q, kc, vc, lens, scale, kn, vn, return_lse=True)
        lens += 1
        if step in (0, 64, 128, 192, 255):
            idx = torch.tensor(picks, device="cuda")
            o_ref, lse_ref = orc.decode_fwd(q[idx].cpu(), kc[idx].cpu(), vc[idx].cpu(), lens[idx].cpu(), scale)
            check_fwd(o[idx], lse[idx], o_ref, lse_ref)
            assert torch.isfinite(o).all()
    assert ext.device_status() == 0
    del kc, vc
    torch.cuda.empty_cache()


# ---------------------------------------------------------------------------------------------
# Long context (single GPU, sampled oracle)
# ---------------------------------------------------------------------------------------------
def _rows_closed_form(q_rows, g_rows, kf, vf, scale, r0, r1):
    """fp32 statistics of query rows [r0, r1) of a causal problem against keys [0, r1): the probabilities
    P, dS = P o (dP - rowsum(dO o O)) and the rows' own O (the closed form of ref_backward,
    tests/test_flash_attn.py:35-58 of the reference, restricted to a row block)."""
    s = torch.matmul(q_rows, kf.transpose(-1, -2)) * scale
    rows = torch.arange(r0, r1).view(-1, 1)
    s.masked_fill_(torch.arange(kf.shape[2]).view(1, -1) > rows, float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.matmul(p, vf)
    ds = p * (torch.matmul(g_rows, vf.transpose(-1, -2)) - (g_rows * o).sum(-1, keepdim=True))
    return p, ds


def test_config5_long_context_sampled(ext):
    """B=1, Hq=32, Hkv=8, N=131072, d=128, causal forward + backward on one GPU.  One score matrix row
    block of one head is 0.5 GB in fp32, so the oracle checks O, LSE and dQ on sampled 256-row blocks
    of one KV-head group (dQ rows depend only on their own row block), dK and dV of the group's LAST
    256 keys (they depend only on the last 256 query rows), and dK and dV of a 256-key block three
    quarters into the sequence, for which a second backward is run with dO zeroed outside one query
    head -- that block's gradient then comes from that head's 32 896 later rows alone, which the
    oracle can afford."""
    B, Hq, Hkv, N, d = 1, 32, 8, 131072, 128
    gen = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn(B, Hq, N, d, device="cuda", generator=gen).half()
    k = torch.randn(B, Hkv, N, d, device="cuda", generator=gen).half()
    v = torch.randn(B, Hkv, N, d, device="cuda", generator=gen).half()
    do = torch.randn(B, Hq, N, d, device="cuda", generator=gen).half()
    scale = 1 / math.sqrt(d)
    o, lse = ext.forward(q, k, v, scale, True)
    dq, dk, dv = ext.backward(do, q, k, v, o, lse, scale, True)
    assert ext.device_status() == 0
    for t in (o, lse, dq, dk, dv):
        assert torch.isfinite(t).all()
    h = 6  # KV head; query heads 24..27
    sl = slice(4 * h, 4 * h + 4)
    kh, vh = k[:, h:h + 1].cpu(), v[:, h:h + 1].cpu()
    for r0 in (0, 65536 - 128, N - 256):
        r1 = r0 + 256
        qs = q[:, sl, :r1].cpu()  # rows beyond r1 are not needed by a causal row block
        o_ref, lse_ref = orc.attention_fwd_rows(qs, kh, vh, scale, True, r0, r1)
        check_fwd(o[:, sl, r0:r1], lse[:, sl, r0:r1], o_ref, lse_ref)
        # dQ of the block: closed form on the block's rows
        kf, vf = kh[:, :, :r1].float(), vh[:, :, :r1].float()
        qf, gf = q[:, sl, r0:r1].cpu().float(), do[:, sl, r0:r1].cpu().float()
        p, ds = _rows_closed_form(qf, gf, kf, vf, scale, r0, r1)
        dq_ref = torch.matmul(ds, kf) * scale
        assert orc.rel_max_err(dq[:, sl, r0:r1], dq_ref) <= orc.TOL_GRAD
        if r1 == N:
            # the last 256 keys are seen by the last 256 queries only: their dK / dV in closed form,
            # summed over the group's four query heads
            dk_ref = (torch.matmul(ds[..., r0:r1].transpose(-1, -2), qf) * scale).sum(1, keepdim=True)
            dv_ref = torch.matmul(p[..., r0:r1].transpose(-1, -2), gf).sum(1, keepdim=True)
            assert orc.rel_max_err(dk[:, h:h + 1, r0:r1], dk_ref) <= orc.TOL_GRAD
            assert orc.rel_max_err(dv[:, h:h + 1, r0:r1], dv_ref) <= orc.TOL_GRAD

    # ---- a key block in mid-sequence: gradient through ONE query head ------------------------
    hq = 4 * h + 1
    do_one = torch.zeros_like(do)
    do_one[:, hq] = do[:, hq]
    _, dk1, dv1 = ext.backward(do_one, q, k, v, o, lse, scale, True)
    assert ext.device_status() == 0
    kb0, kb1 = 98176, 98432
    qh, gh = q[:, hq:hq + 1].cpu().float(), do[:, hq:hq + 1].cpu().float()
    kf, vf = kh.float(), vh.float()
    dk_ref = torch.zeros(1, 1, kb1 - kb0, d)
    dv_ref = torch.zeros(1, 1, kb1 - kb0, d)
    for r0 in range(kb0, N, 1024):   # rows before kb0 do not see the block
        r1 = min(N, r0 + 1024)
        p, ds = _rows_closed_form(qh[:, :, r0:r1], gh[:, :, r0:r1], kf[:, :, :r1], vf[:, :, :r1], scale, r0, r1)
        dk_ref += torch.matmul(ds[..., kb0:kb1].transpose(-1, -2), qh[:, :, r0:r1]) * scale
        dv_ref += torch.matmul(p[..., kb0:kb1].transpose(-1, -2), gh[:, :, r0:r1])
    assert orc.rel_max_err(dk1[:, h:h + 1, kb0:kb1], dk_ref) <= orc.TOL_GRAD
    assert orc.rel_max_err(dv1[:, h:h + 1, kb0:kb1], dv_ref) <= orc.TOL_GRAD
    del q, k, v, do, do_one, o, dq, dk, dv, dk1, dv1
    torch.cuda.empty_cache()


# ---------------------------------------------------------------------------------------------
# The public operator surface (autograd, modules, error behaviour)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d", [32, 64, 96, 128])
def test_flash_attention_autograd_all_head_dims(fal, d):
    g = torch.Generator().manual_seed(30 + d)
    q, k, v, do = rand_half(g, 1, 4, 130, d), rand_half(g, 1, 2, 130, d), rand_half(g, 1, 2, 130, d), rand_half(g, 1, 4, 130, d)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = fal.flash_attention(qc, kc, vc, is_causal=True)
    assert out.shape == q.shape and out.dtype == torch.float16
    out.backward(do.cuda())
    scale = 1 / math.sqrt(d)
    o_ref, _ = orc.attention_fwd(q, k, v, scale, True)
    assert orc.rel_max_err(out.detach(), o_ref) <= orc.TOL_O
    check_grads((qc.grad, kc.grad, vc.grad), orc.attention_bwd(q, k, v, do, scale, True))


@pytest.mark.parametrize("causal", [False, True])
def test_operator_reads_strided_views_and_writes_bnhd_memory(fal, causal):
    """The layout a transformer block has: [B,N,H,d] projections viewed as [B,H,N,d], and an output the
    block transposes back.  Neither side of the operator should need a copy, forward or backward."""
    gen = torch.Generator().manual_seed(21)
    b, hq, hkv, n, d = 2, 8, 2, 300, 128
    q_mem, k_mem, v_mem = rand_half(gen, b, n, hq, d), rand_half(gen, b, n, hkv, d), rand_half(gen, b, n, hkv, d)
    do_mem = rand_half(gen, b, n, hq, d)
    q, k, v = (t.cuda().transpose(1, 2).requires_grad_(True) for t in (q_mem, k_mem, v_mem))
    assert not q.is_contiguous()
    scale = 1.0 / math.sqrt(d)
    out = fal.flash_attention(q, k, v, softmax_scale=scale, is_causal=causal, out_layout="bnhd")
    assert out.shape == (b, hq, n, d) and out.transpose(1, 2).is_contiguous()
    out.backward(do_mem.cuda().transpose(1, 2))  # a strided gradient, as the block's reshape produces
    qf, kf, vf, dof = (t.transpose(1, 2).contiguous() for t in (q_mem, k_mem, v_mem, do_mem))
    o_ref, _ = orc.attention_fwd(qf, kf, vf, scale, causal)
    assert orc.rel_max_err(out, o_ref) <= orc.TOL_O
    check_grads((q.grad, k.grad, v.grad), orc.attention_bwd(qf, kf, vf, dof, scale, causal))
    # default layout unchanged: contiguous [B,H,N,d]
    assert fal.flash_attention(q.detach(), k.detach(), v.detach(), is_causal=causal).is_contiguous()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("n", [1, 200, 1000])
def test_head_dim_256_forward(ext, causal, n):
    """head_dim 256 forward: one 128-row query tile per CTA."""
    gen = torch.Generator().manual_seed(n)
    b, hq, hkv, d = 2, 4, 2, 256
    q, k, v = rand_half(gen, b, hq, n, d), rand_half(gen, b, hkv, n, d), rand_half(gen, b, hkv, n, d)
    scale = 1.0 / math.sqrt(d)
    o, lse = ext.forward(q.cuda(), k.cuda(), v.cuda(), scale, causal)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, scale, causal)
    if n == 1:
        assert torch.equal(o.cpu(), v.repeat_interleave(hq // hkv, 1))
    else:
        check_fwd(o, lse, o_ref, lse_ref)
    assert ext.device_status() == 0


def test_head_dim_256_varlen_forward_and_decode(ext):
    gen = torch.Generator().manual_seed(8)
    lens = [300, 17, 520]
    total, hq, hkv, d = sum(lens), 4, 2, 256
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    q, k, v = rand_half(gen, total, hq, d), rand_half(gen, total, hkv, d), rand_half(gen, total, hkv, d)
    o, lse = ext.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens), 0.07, True)
    o_ref, lse_ref = orc.varlen_fwd(q, k, v, cu, cu, 0.07, True)
    check_fwd(o, lse, o_ref, lse_ref)

    b, cap = 3, 2048
    kc, vc = rand_half(gen, b, cap, hkv, d), rand_half(gen, b, cap, hkv, d)
    qd = rand_half(gen, b, hq, d)
    seqlens = torch.tensor([1, 1500, 2048], dtype=torch.int32)
    out = ext.decode(qd.cuda(), kc.cuda(), vc.cuda(), seqlens.cuda(), 0.07)
    out = out[0] if isinstance(out, (list, tuple)) else out
    ref = orc.decode_fwd(qd, kc, vc, seqlens, 0.07)
    ref = ref[0] if isinstance(ref, (list, tuple)) else ref
    assert orc.rel_max_err(out, ref) <= orc.TOL_O
    assert ext.device_status() == 0


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("n", [1, 64, 200, 513])
def test_head_dim_256_backward(ext, causal, n):
    """head_dim 256 backward: two CTAs per key tile, 128 columns of dQ, dK and dV each, GQA 2:1."""
    gen = torch.Generator().manual_seed(256 + n)
    b, hq, hkv, d = 2, 4, 2, 256
    q, k, v, do = (rand_half(gen, b, hq, n, d), rand_half(gen, b, hkv, n, d), rand_half(gen, b, hkv, n, d),
                   rand_half(gen, b, hq, n, d))
    scale = 1.0 / math.sqrt(d)
    o, lse, grads = run_fwd_bwd(ext, q, k, v, do, scale, causal)
    assert ext.device_status() == 0
    ref = orc.attention_bwd(q, k, v, do, scale, causal)
    if n == 1:
        assert grads[0].abs().max().item() < 1e-3 and grads[1].abs().max().item() < 1e-3
        assert orc.rel_max_err(grads[2], ref[2]) <= orc.TOL_GRAD
    else:
        check_grads(grads, ref)


def test_head_dim_256_varlen_backward_and_autograd(ext, fal):
    gen = torch.Generator().manual_seed(77)
    lens = [300, 17, 0, 140]
    q, k, v, do, cu = packed_inputs(gen, lens, 4, 2, 256)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = fal.flash_attn_varlen_func(qc, kc, vc, cu.cuda(), cu.cuda(), 300, 300, causal=True)
    out.backward(do.cuda())
    check_grads((qc.grad, kc.grad, vc.grad), orc.varlen_bwd(q, k, v, do, cu, cu, 1 / 16, True))
    # the batched operator through autograd, strided [B,N,H,d] inputs
    xq, xk, xv = (torch.randn(1, 150, 2, 256, generator=gen).half() for _ in range(3))
    g = torch.randn(1, 2, 150, 256, generator=gen).half()
    tq, tk, tv = (t.cuda().requires_grad_(True) for t in (xq, xk, xv))
    y = fal.flash_attention(tq.transpose(1, 2), tk.transpose(1, 2), tv.transpose(1, 2), is_causal=True)
    y.backward(g.cuda())
    ref = orc.attention_bwd(xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2), g, 1 / 16, True)
    check_grads((tq.grad.transpose(1, 2), tk.grad.transpose(1, 2), tv.grad.transpose(1, 2)), ref)
    assert ext.device_status() == 0


@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("nq,nk", [(1, 300), (100, 100), (128, 512), (200, 777), (257, 1000), (513, 514)])
def test_forward_with_the_causal_mask_aligned_to_the_end_of_the_keys(ext, d, nq, nk):
    """A chunk of new tokens behind a cached prefix: query i sees keys j <= i + nk - nq."""
    gen = torch.Generator().manual_seed(nq * 3 + nk + d)
    b, hq, hkv = 2, 4, 2
    q, k, v = rand_half(gen, b, hq, nq, d), rand_half(gen, b, hkv, nk, d), rand_half(gen, b, hkv, nk, d)
    scale = 1.0 / math.sqrt(d)
    o, lse = ext.forward_rect(q.cuda(), k.cuda(), v.cuda(), scale, True, bottom_right=True)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, scale, True, causal_shift=nk - nq)
    check_fwd(o, lse, o_ref, lse_ref)
    assert ext.device_status() == 0
    if nk > nq:  # more queries than keys: the alignment is not defined, the call is refused
        with pytest.raises(RuntimeError):
            ext.forward_rect(k.cuda(), q[:, :hkv].cuda(), q[:, :hkv].cuda(), scale, True, bottom_right=True)


@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("nq,nk", [(1, 300), (100, 100), (128, 512), (200, 777), (257, 1000), (640, 700)])
def test_backward_with_the_causal_mask_aligned_to_the_end_of_the_keys(ext, d, nq, nk):
    """Gradients of a chunk of new tokens behind a cached prefix (query i sees keys j <= i + nk - nq)."""
    gen = torch.Generator().manual_seed(nq * 5 + nk + d)
    b, hq, hkv = 2, 4, 2
    q, k, v, do = (rand_half(gen, b, hq, nq, d), rand_half(gen, b, hkv, nk, d), rand_half(gen, b, hkv, nk, d),
                   rand_half(gen, b, hq, nq, d))
    scale = 1.0 / math.sqrt(d)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o, lse = ext.forward_rect(qc, kc, vc, scale, True, bottom_right=True)
    grads = ext.backward(do.cuda(), qc, kc, vc, o, lse, scale, True, bottom_right=True)
    ref = orc.attention_bwd(q, k, v, do, scale, True, causal_shift=nk - nq)
    if nq == 1 and nk == 1:
        return
    check_grads(grads, ref)
    assert ext.device_status() == 0
    with pytest.raises(RuntimeError):   # fewer keys than queries: the alignment is not defined
        ext.backward(do.cuda(), qc, kc[:, :, :max(nq - 1, 0)], vc[:, :, :max(nq - 1, 0)], o, lse, scale, True,
                     bottom_right=True)


@pytest.mark.parametrize("d,h,hkv", [(64, 4, 4), (128, 8, 2)])
def test_varlen_with_end_aligned_masks_forward_and_backward(ext, d, h, hkv):
    """Packed sequences whose queries are the LAST len_q positions of their len_k keys: ragged chunks
    behind ragged prefixes.  One sequence has more queries than keys (its first rows see nothing)."""
    gen = torch.Generator().manual_seed(77 + d)
    lq, lk = [40, 130, 7, 256, 50, 1], [100, 130, 300, 1000, 20, 129]
    cu_q = torch.tensor([0] + list(torch.tensor(lq).cumsum(0)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(lk).cumsum(0)), dtype=torch.int32)
    q, do = rand_half(gen, sum(lq), h, d), rand_half(gen, sum(lq), h, d)
    k, v = rand_half(gen, sum(lk), hkv, d), rand_half(gen, sum(lk), hkv, d)
    scale = 1.0 / math.sqrt(d)
    o, lse = ext.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), max(lq), max(lk), scale,
                                True, bottom_right=True)
    o_ref, lse_ref = orc.varlen_fwd(q, k, v, cu_q, cu_k, scale, True, bottom_right=True)
    check_fwd(o, lse, o_ref, lse_ref)
    grads = ext.backward_varlen(do.cuda(), q.cuda(), k.cuda(), v.cuda(), o, lse, cu_q.cuda(), cu_k.cuda(), max(lq),
                                max(lk), scale, True, bottom_right=True)
    check_grads(grads, orc.varlen_bwd(q, k, v, do, cu_q, cu_k, scale, True, bottom_right=True))
    assert ext.device_status() == 0


@pytest.mark.parametrize("d", [32, 96])
def test_head_dims_32_and_96_run_without_padded_copies(ext, fal, d):
    """32 and 96 run on the 64 / 128 kernels: the TMA descriptors carry the real width (the missing
    columns arrive as zeros) and no output column beyond it is written.  Batched forward + backward
    (both forward variants), packed, chunk, decode with append -- straight through the binding, into
    output tensors with guard columns that must stay untouched."""
    gen = torch.Generator().manual_seed(1000 + d)
    scale = 1.0 / math.sqrt(d)
    # batched, strided [B,N,H,d] inputs, both forward variants
    b, hq, hkv, n = 2, 4, 2, 333
    qm, km, vm, dom = rand_half(gen, b, n, hq, d), rand_half(gen, b, n, hkv, d), rand_half(gen, b, n, hkv, d), rand_half(gen, b, n, hq, d)
    q, k, v, do = (t.cuda().transpose(1, 2) for t in (qm, km, vm, dom))
    qf, kf, vf, dof = (t.transpose(1, 2) for t in (qm, km, vm, dom))
    o_ref, lse_ref = orc.attention_fwd(qf, kf, vf, scale, True)
    ref = orc.attention_bwd(qf, kf, vf, dof, scale, True)
    for variant in (1, 2):
        ext.set_forward_variant(variant)
        try:
            wide = torch.full((b, hq, n, d + 8), 7.0, dtype=torch.float16, device="cuda")   # guard columns
            o, lse = ext.forward(q, k, v, scale, True, out=wide[..., :d])
        finally:
            ext.set_forward_variant(0)
        check_fwd(o, lse, o_ref, lse_ref)
        assert (wide[..., d:] == 7.0).all()
    gw = [torch.full((b, h, n, d + 8), 7.0, dtype=torch.float16, device="cuda") for h in (hq, hkv, hkv)]
    grads = ext.backward(do, q, k, v, o, lse, scale, True, out=[t[..., :d] for t in gw])
    check_grads(grads, ref)
    assert all((t[..., d:] == 7.0).all() for t in gw)
    # packed, through the autograd operator
    lens = [70, 300, 9]
    qp, kp, vp, dop, cu = packed_inputs(gen, lens, 4, 2, d)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (qp, kp, vp))
    out = fal.flash_attn_varlen_func(qc, kc, vc, cu.cuda(), cu.cuda(), 300, 300, causal=True)
    out.backward(dop.cuda())
    o_ref, _ = orc.varlen_fwd(qp, kp, vp, cu, cu, scale, True)
    assert orc.rel_max_err(out.detach(), o_ref) <= orc.TOL_O
    check_grads((qc.grad, kc.grad, vc.grad), orc.varlen_bwd(qp, kp, vp, dop, cu, cu, scale, True))
    # a chunk behind a prefix
    qx, kx, vx = rand_half(gen, 1, 4, 100, d), rand_half(gen, 1, 2, 420, d), rand_half(gen, 1, 2, 420, d)
    oc = fal.flash_attention_chunk(qx.cuda(), kx.cuda(), vx.cuda())
    assert orc.rel_max_err(oc, orc.attention_fwd(qx, kx, vx, scale, True, causal_shift=320)[0]) <= orc.TOL_O
    # decode with an append, both cache layouts
    B, S = 3, 1500
    kc_, vc_, qd = rand_half(gen, B, S, hkv, d), rand_half(gen, B, S, hkv, d), rand_half(gen, B, hq, d)
    kn, vn = rand_half(gen, B, hkv, d), rand_half(gen, B, hkv, d)
    lens_t = torch.tensor([0, 1023, 1499], dtype=torch.int32)
    for layout in ("bshd", "bhsd"):
        kcc, vcc = kc_.cuda(), vc_.cuda()
        if layout == "bhsd":
            kcc, vcc = kcc.transpose(1, 2).contiguous(), vcc.transpose(1, 2).contiguous()
        od, lsed = ext.decode(qd.cuda(), kcc, vcc, lens_t.cuda(), scale, kn.cuda(), vn.cuda(), cache_layout=layout,
                              return_lse=True)
        kr, vr = kc_.clone(), vc_.clone()
        for i in range(B):
            kr[i, lens_t[i]], vr[i, lens_t[i]] = kn[i], vn[i]
        got_k = kcc if layout == "bshd" else kcc.transpose(1, 2)
        assert torch.equal(got_k.cpu(), kr)
        check_fwd(od, lsed, *orc.decode_fwd(qd, kr, vr, lens_t + 1, scale))
    assert ext.device_status() == 0


def test_chunked_prefill_equals_one_prefill(fal):
    """Prefill in three chunks through flash_attention_chunk == one causal flash_attention call."""
    gen = torch.Generator().manual_seed(99)
    b, hq, hkv, n, d = 1, 8, 2, 700, 128
    q, k, v = (rand_half(gen, b, hq, n, d).cuda(), rand_half(gen, b, hkv, n, d).cuda(),
               rand_half(gen, b, hkv, n, d).cuda())
    whole = fal.flash_attention(q, k, v, is_causal=True)
    parts, start = [], 0
    for size in (256, 300, 144):
        end = start + size
        parts.append(fal.flash_attention_chunk(q[:, :, start:end], k[:, :, :end], v[:, :, :end]))
        start = end
    chunked = torch.cat(parts, dim=2)
    assert orc.rel_max_err(chunked, whole.float().cpu()) <= orc.TOL_O
    out = fal.flash_attention_chunk(q[:, :, -50:], k, v, out_layout="bnhd")
    assert out.transpose(1, 2).is_contiguous()
    assert orc.rel_max_err(out, whole[:, :, -50:].float().cpu()) <= orc.TOL_O
    # and it is differentiable: the gradients of the last 300 positions against the oracle
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q[:, :, -300:], k, v))
    do = rand_half(gen, b, hq, 300, d).cuda()
    fal.flash_attention_chunk(qg, kg, vg).backward(do)
    ref = orc.attention_bwd(q[:, :, -300:].cpu(), k.cpu(), v.cpu(), do.cpu(), 1 / math.sqrt(d), True, causal_shift=n - 300)
    check_grads((qg.grad, kg.grad, vg.grad), ref)


@pytest.mark.parametrize("layout", ["bshd", "bhsd"])
@pytest.mark.parametrize("d", [64, 128])
def test_chunk_against_caches_of_different_lengths(ext, fal, layout, d):
    """A chunk of new tokens per entry against caches filled to different lengths (fal_fwd_kvcache):
    through the binding with the chunk already in the caches, and through flash_attn_with_kvcache, which
    appends it first.  What lies behind an entry's length is NaN / infinity here and must not matter."""
    gen = torch.Generator().manual_seed(41 + d)
    B, Hq, Hkv, S = 5, 8, 2, 1000
    scale = 1 / math.sqrt(d)
    for lq, lens in ((37, [1000, 37, 128, 513, 64]), (256, [256, 999, 300, 640, 257]), (130, [130, 131, 1000, 258, 500])):
        lens_t = torch.tensor(lens, dtype=torch.int32)
        kc, vc = rand_half(gen, B, Hkv, S, d), rand_half(gen, B, Hkv, S, d)
        for b in range(B):
            kc[b, :, lens[b]:] = float("nan")
            vc[b, :, lens[b]:] = float("inf")
        q = rand_half(gen, B, Hq, lq, d)
        o_ref, lse_ref = orc.kvcache_chunk_fwd(q, kc, vc, lens_t, scale)
        kc_dev = kc.cuda() if layout == "bhsd" else kc.transpose(1, 2).contiguous().cuda()   # [B,S,Hkv,d] memory
        vc_dev = vc.cuda() if layout == "bhsd" else vc.transpose(1, 2).contiguous().cuda()
        kv_view = (lambda t: t) if layout == "bhsd" else (lambda t: t.transpose(1, 2))
        o, lse = ext.forward_kvcache(q.cuda(), kv_view(kc_dev), kv_view(vc_dev), lens_t.cuda(), scale)
        check_fwd(o, lse, o_ref, lse_ref)
        # the operator: the caches hold everything but the chunk, which it appends
        old = lens_t - lq
        k_new = torch.stack([kc[b, :, old[b]:lens[b]] for b in range(B)]).transpose(1, 2).contiguous()   # [B,lq,Hkv,d]
        v_new = torch.stack([vc[b, :, old[b]:lens[b]] for b in range(B)]).transpose(1, 2).contiguous()
        for b in range(B):
            kc_dev_b = kv_view(kc_dev)[b]
            kc_dev_b[:, int(old[b]):int(lens[b])] = float("nan")        # not there yet
        out = fal.flash_attn_with_kvcache(q.transpose(1, 2).contiguous().cuda(), kc_dev, vc_dev, k_new.cuda(), v_new.cuda(),
                                          cache_seqlens=old.cuda(), cache_layout=layout)
        assert tuple(out.shape) == (B, lq, Hq, d)
        assert orc.rel_max_err(out.transpose(1, 2), o_ref) <= orc.TOL_O
        for b in range(B):     # and the chunk is in the caches now
            assert torch.equal(kv_view(kc_dev)[b, :, int(old[b]):lens[b]].cpu(), kc[b, :, int(old[b]):lens[b]])
    # an entry shorter than the chunk: its first queries see no key
    lens_t = torch.tensor([10, 200, 0, 64, 65], dtype=torch.int32)
    kc, vc, q = rand_half(gen, B, Hkv, S, d), rand_half(gen, B, Hkv, S, d), rand_half(gen, B, Hq, 64, d)
    o, lse = ext.forward_kvcache(q.cuda(), kc.cuda(), vc.cuda(), lens_t.cuda(), scale)
    check_fwd(o, lse, *orc.kvcache_chunk_fwd(q, kc, vc, lens_t, scale))
    assert ext.device_status() == 0


def test_broadcast_views_are_copied_not_misread(ext, fal):
    """K/V expanded over the heads (stride 0) and the expanded gradient of a reduction: the operator
    copies them, the binding refuses them (tests/test_flash_attn.py:177-193 of the reference)."""
    gen = torch.Generator().manual_seed(12)
    b, hq, n, d = 2, 8, 128, 64
    q, k, v = (rand_half(gen, b, hq, n, d).cuda(), rand_half(gen, b, 1, n, d).cuda(),
               rand_half(gen, b, 1, n, d).cuda())
    mqa = fal.flash_attention(q, k, v)
    mha = fal.flash_attention(q, k.expand(b, hq, n, d), v.expand(b, hq, n, d))
    assert torch.equal(mqa, mha)
    with pytest.raises(RuntimeError):
        ext.forward(q, k.expand(b, hq, n, d), v.expand(b, hq, n, d), 0.125, False)
    # gradient of out.sum(dim=2): every row gets the same [B,H,1,d] slice, expanded along the rows
    qg = q.clone().requires_grad_(True)
    w = rand_half(gen, b, hq, d).cuda()
    (fal.flash_attention(qg, k, v, is_causal=True).sum(dim=2) * w).sum().backward()
    do = w[:, :, None, :].expand(b, hq, n, d).contiguous()
    ref = orc.attention_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), 0.125, True)
    assert orc.rel_max_err(qg.grad, ref[0]) <= orc.TOL_GRAD


def test_varlen_func_autograd(fal):
    g = torch.Generator().manual_seed(31)
    lens = [70, 130, 9]
    q, k, v, do, cu = packed_inputs(g, lens, 4, 4, 64)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = fal.flash_attn_varlen_func(qc, kc, vc, cu.cuda(), cu.cuda(), 130, 130, causal=True)
    out.backward(do.cuda())
    o_ref, _ = orc.varlen_fwd(q, k, v, cu, cu, 0.125, True)
    assert orc.rel_max_err(out.detach(), o_ref) <= orc.TOL_O
    check_grads((qc.grad, kc.grad, vc.grad), orc.varlen_bwd(q, k, v, do, cu, cu, 0.125, True))


def test_operator_rejects_what_the_reference_rejects(fal):
    q = torch.zeros(1, 2, 16, 64, device="cuda")
    with pytest.raises(AssertionError):
        fal.flash_attention(q, q, q)  # float32
    qh = torch.zeros(1, 2, 16, 80, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError):
        fal.flash_attention(qh, qh, qh)  # head_dim 80
    qh = torch.zeros(1, 3, 16, 64, device="cuda", dtype=torch.float16)
    kh = torch.zeros(1, 2, 16, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError):
        fal.flash_attention(qh, kh, kh)  # 3 % 2 != 0
    with pytest.raises((AssertionError, RuntimeError)):
        fal.flash_attention(qh.cpu(), qh.cpu(), qh.cpu())


def test_modules(fal):
    torch.manual_seed(0)
    mha = fal.FlashMultiHeadAttention(256, num_heads=4, num_kv_heads=2, causal=True).cuda()
    x = torch.randn(2, 50, 256, device="cuda", requires_grad=True)
    y = mha(x)
    assert y.shape == x.shape and y.dtype == x.dtype
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    attn = fal.FlashAttention(head_dim=64, causal=True)
    q = torch.randn(1, 2, 40, 64, device="cuda", dtype=torch.float16)
    assert attn(q, q, q).shape == q.shape


def test_utils(fal):
    info = fal.get_device_info()
    assert info["supported"] and info["sm_version"] // 10 == 10
    assert fal.check_gpu_compatibility(verbose=False)


# ---------------------------------------------------------------------------------------------
# HuggingFace route: attn_implementation="flash_attn_legacy" on a tiny random LLaMA
# ---------------------------------------------------------------------------------------------
def _tiny_llama(attn):
    transformers = pytest.importorskip("transformers")
    cfg = transformers.LlamaConfig(vocab_size=1000, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=8, num_key_value_heads=2, max_position_embeddings=512)
    torch.manual_seed(0)
    cfg._attn_implementation = attn
    return transformers.LlamaForCausalLM(cfg).half().cuda().eval()


def test_hf_registration_prefill_and_generate(fal):
    assert fal.register()
    ref_model = _tiny_llama("eager")
    model = _tiny_llama("flash_attn_legacy")
    model.load_state_dict(ref_model.state_dict())
    assert model.config._attn_implementation == "flash_attn_legacy"
    ids = torch.randint(0, 1000, (2, 64), device="cuda")
    with torch.no_grad():
        a = model(ids).logits.float()
        b = ref_model(ids).logits.float()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.999
    # one cached decode step: logits must agree with eager attention on the same cache
    with torch.no_grad():
        pre = model(ids[:, :40], use_cache=True)
        pre_ref = ref_model(ids[:, :40], use_cache=True)
        step = model(ids[:, 40:41], past_key_values=pre.past_key_values, use_cache=True).logits.float()
        step_ref = ref_model(ids[:, 40:41], past_key_values=pre_ref.past_key_values, use_cache=True).logits.float()
    cos = torch.nn.functional.cosine_similarity(step.flatten(), step_ref.flatten(), dim=0).item()
    assert cos > 0.999
    import flash_attn_legacy_cuda as ext
    ext.profile_enable(True)
    ext.profile_read(ext.KERNEL_DECODE_SPLITK)
    with torch.no_grad():
        out = model.generate(ids[:, :8], max_new_tokens=16, do_sample=False)
    _, launches = ext.profile_read(ext.KERNEL_DECODE_SPLITK)
    ext.profile_enable(False)
    assert out.shape == (2, 24)
    assert launches >= 15 * 2  # every decode step of both layers ran the split-K kernel


def test_hf_chunk_of_new_tokens_against_a_cache(fal):
    """24 new tokens after a cached prefix of 40: the hook runs the forward kernel with the causal
    mask aligned to the end of the cache, and agrees with eager attention (which gets transformers'
    explicit mask for this case)."""
    assert fal.register()
    ref_model = _tiny_llama("eager")
    model = _tiny_llama("flash_attn_legacy")
    model.load_state_dict(ref_model.state_dict())
    ids = torch.randint(0, 1000, (2, 64), device="cuda")
    import flash_attn_legacy_cuda as ext
    with torch.no_grad():
        pre = model(ids[:, :40], use_cache=True)
        pre_ref = ref_model(ids[:, :40], use_cache=True)
        ext.profile_enable(True)
        ext.profile_read(ext.KERNEL_FWD)
        chunk = model(ids[:, 40:], past_key_values=pre.past_key_values, use_cache=True).logits.float()
        _, launches = ext.profile_read(ext.KERNEL_FWD)
        ext.profile_enable(False)
        chunk_ref = ref_model(ids[:, 40:], past_key_values=pre_ref.past_key_values, use_cache=True).logits.float()
        whole = ref_model(ids).logits.float()[:, 40:]
    assert launches == 2  # one forward-kernel launch per layer, no eager fallback
    cos = torch.nn.functional.cosine_similarity(chunk.flatten(), chunk_ref.flatten(), dim=0).item()
    assert cos > 0.999
    cos = torch.nn.functional.cosine_similarity(chunk.flatten(), whole.flatten(), dim=0).item()
    assert cos > 0.999


def test_llama_patch_route(fal):
    """The reference's second integration route (examples/hf_llama_patch.py: replace every
    LlamaAttention.forward) on a tiny random LLaMA, as its tests/test_transformers.py does."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "flash-attention-legacy_b200",
                        "examples", "hf_llama_patch.py")
    spec = importlib.util.spec_from_file_location("hf_llama_patch", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    ref_model = _tiny_llama("eager")
    model = _tiny_llama("eager")
    model.load_state_dict(ref_model.state_dict())
    assert mod.patch_llama_attention(model) is model
    ids = torch.randint(0, 1000, (2, 64), device="cuda")
    import flash_attn_legacy_cuda as ext
    ext.profile_enable(True)
    ext.profile_read(ext.KERNEL_FWD)
    with torch.no_grad():
        a = model(ids).logits.float()
        b = ref_model(ids).logits.float()
    _, launches = ext.profile_read(ext.KERNEL_FWD)
    ext.profile_enable(False)
    assert launches == 2
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.999
    with torch.no_grad():
        out = model.generate(ids[:, :8], max_new_tokens=12, do_sample=False)
        out_ref = ref_model.generate(ids[:, :8], max_new_tokens=12, do_sample=False)
    assert out.shape == (2, 20)
    assert (out == out_ref).float().mean().item() > 0.8  # greedy tokens of random weights: near-ties may flip


def test_hf_padded_batch_runs_unpadded_through_the_packed_kernels(fal):
    from flash_attn_legacy.integrations import _padded_prefill
    gen = torch.Generator().manual_seed(5)
    b, hq, hkv, n, d = 3, 8, 2, 200, 128
    q, k, v = rand_half(gen, b, hq, n, d), rand_half(gen, b, hkv, n, d), rand_half(gen, b, hkv, n, d)
    keep = torch.ones(b, n, dtype=torch.bool)
    keep[0, :37] = False          # left padding
    keep[1, 150:] = False         # right padding
    scale = 1.0 / math.sqrt(d)
    out = _padded_prefill(q.cuda(), k.cuda(), v.cuda(), keep.cuda(), scale, True)  # [B, N, Hq, d]
    assert out.shape == (b, n, hq, d)
    for row in range(b):
        sel = keep[row]
        o_ref, _ = orc.attention_fwd(q[row:row + 1, :, sel], k[row:row + 1, :, sel], v[row:row + 1, :, sel], scale, True)
        got = out[row, sel.cuda()].transpose(0, 1).unsqueeze(0)
        assert orc.rel_max_err(got, o_ref) <= orc.TOL_O
        assert (out[row, (~sel).cuda()] == 0).all()

    # the whole route: a left-padded batch through a tiny LLaMA against eager attention
    assert fal.register()
    ref_model = _tiny_llama("eager")
    model = _tiny_llama("flash_attn_legacy")
    model.load_state_dict(ref_model.state_dict())
    ids = torch.randint(0, 1000, (2, 48), device="cuda")
    mask = torch.ones(2, 48, dtype=torch.long, device="cuda")
    mask[1, :17] = 0
    import flash_attn_legacy_cuda as ext
    with torch.no_grad():
        a = model(ids, attention_mask=mask).logits.float()
        r = ref_model(ids, attention_mask=mask).logits.float()
    real = mask.bool()
    cos = torch.nn.functional.cosine_similarity(a[real].flatten(), r[real].flatten(), dim=0).item()
    assert cos > 0.999
    ext.profile_enable(True)
    ext.profile_read(ext.KERNEL_DECODE_SPLITK)
    with torch.no_grad():
        out = model.generate(ids[:, :24], attention_mask=mask[:, :24], max_new_tokens=8, do_sample=False)
        out_ref = ref_model.generate(ids[:, :24], attention_mask=mask[:, :24], max_new_tokens=8, do_sample=False)
    _, decode_launches = ext.profile_read(ext.KERNEL_DECODE_SPLITK)
    ext.profile_enable(False)
    assert decode_launches >= 7 * 2  # the decode steps of the left-padded batch ran the split-K kernel
    assert out.shape == (2, 32)
    assert (out == out_ref).float().mean().item() > 0.9  # greedy tokens agree (fp16 ties aside)
    assert ext.device_status() == 0
