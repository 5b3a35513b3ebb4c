"""CPU: the oracle against the golden vectors produced by the reference's own code, and against
the reference's known-answer tests (tests/test_flash_attn.py of sirCamp/flash-attention-legacy)."""
import math

import pytest
import torch

from conftest import golden_names, load_golden
from oracle import attention_oracle as orc

# The golden outputs are fp16 (the reference's ref_attention / ref_backward end in .half()).
HALF_EPS = 2.0 ** -10


def _close_to_half(x32, ref16, what):
    ref = ref16.float()
    tol = HALF_EPS * ref.abs().max().item() + 1e-6
    err = (x32 - ref).abs().max().item()
    assert err <= tol, f"{what}: max abs err {err} > {tol}"


@pytest.mark.parametrize("name", golden_names("batched_"))
def test_batched_forward_backward_match_reference_vectors(name):
    g = load_golden(name)
    o, _ = orc.attention_fwd(g["q"], g["k"], g["v"], float(g["scale"]), bool(g["causal"]))
    _close_to_half(o, g["o"], "O")
    dq, dk, dv = orc.attention_bwd(g["q"], g["k"], g["v"], g["d_out"], float(g["scale"]), bool(g["causal"]))
    _close_to_half(dq, g["dq"], "dQ")
    _close_to_half(dk, g["dk"], "dK")
    _close_to_half(dv, g["dv"], "dV")


@pytest.mark.parametrize("name", golden_names("batched_"))
def test_blocked_variants_equal_unblocked(name):
    g = load_golden(name)
    args = (g["q"], g["k"], g["v"])
    scale, causal = float(g["scale"]), bool(g["causal"])
    o, lse = orc.attention_fwd(*args, scale, causal)
    ob, lb = orc.attention_fwd_blocked(*args, scale, causal, block=37)
    assert (o - ob).abs().max().item() < 1e-5 and (lse - lb).abs().max().item() < 1e-5
    ref = orc.attention_bwd(*args, g["d_out"], scale, causal)
    got = orc.attention_bwd_blocked(*args, g["d_out"], scale, causal, block=37)
    for a, b in zip(got, ref):
        assert (a - b).abs().max().item() < 1e-4 * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("name", golden_names("varlen_"))
def test_varlen_matches_reference_vectors(name):
    g = load_golden(name)
    o, lse = orc.varlen_fwd(g["q"], g["k"], g["v"], g["cu_seqlens"], g["cu_seqlens"], float(g["scale"]),
                            bool(g["causal"]))
    _close_to_half(o, g["o"], "O")
    assert lse.shape == (g["q"].shape[0], g["q"].shape[1]) and torch.isfinite(lse).all()


def test_decode_matches_reference_hook_vectors():
    g = load_golden("decode_hook_d64")
    o, lse = orc.decode_fwd(g["q"], g["k_cache"], g["v_cache"], g["cache_seqlens"], float(g["scale"]))
    assert (o - g["o"].float()).abs().max().item() < 1e-5
    assert torch.isfinite(lse).all()


def test_lse_is_natural_log_of_scaled_scores():
    # Definition pinned by the reference forward kernel: L = m + ln(l) of the scaled, masked scores
    # (csrc/kernels/flash_attn_fwd_volta.cu:343).
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 1, 5, 8), torch.randn(1, 1, 5, 8), torch.randn(1, 1, 5, 8)
    _, lse = orc.attention_fwd(q, k, v, 0.5, True)
    for i in range(5):
        s = (q[0, 0, i] @ k[0, 0, : i + 1].T) * 0.5
        assert abs(lse[0, 0, i].item() - math.log(torch.exp(s).sum().item())) < 1e-5


# ---- the reference's known-answer tests, applied to the oracle ------------------------------------

def test_single_token_returns_v():                      # tests/test_flash_attn.py:111-117
    q, k, v = torch.randn(2, 4, 1, 64), torch.randn(2, 4, 1, 64), torch.randn(2, 4, 1, 64)
    o, _ = orc.attention_fwd(q, k, v, 0.125, True)
    assert torch.allclose(o, v, atol=1e-6)


def test_zero_scores_give_mean_of_v():                  # tests/test_flash_attn.py:119-127
    v = torch.randn(1, 1, 64, 32)
    o, lse = orc.attention_fwd(torch.zeros(1, 1, 64, 32), torch.zeros(1, 1, 64, 32), v, 1.0)
    assert torch.allclose(o, v.mean(dim=2, keepdim=True).expand_as(v), atol=1e-6)
    assert torch.allclose(lse, torch.full_like(lse, math.log(64)), atol=1e-6)


def test_causal_first_row_is_v0():                      # tests/test_flash_attn.py:645-656
    q, k, v = torch.randn(1, 2, 16, 32), torch.randn(1, 2, 16, 32), torch.randn(1, 2, 16, 32)
    o, _ = orc.attention_fwd(q, k, v, 0.2, True)
    assert torch.allclose(o[:, :, 0], v[:, :, 0], atol=1e-6)


def test_mqa_equals_explicit_broadcast():               # tests/test_flash_attn.py:177-193
    q, k, v = torch.randn(1, 4, 20, 32), torch.randn(1, 1, 20, 32), torch.randn(1, 1, 20, 32)
    a, _ = orc.attention_fwd(q, k, v, 0.2, True)
    b, _ = orc.attention_fwd(q, k.expand(1, 4, 20, 32), v.expand(1, 4, 20, 32), 0.2, True)
    assert torch.allclose(a, b, atol=1e-6)


def test_gqa_gradient_shapes_and_group_sum():           # tests/test_flash_attn.py:244-257, :56-57
    q, k, v, g = torch.randn(1, 4, 12, 16), torch.randn(1, 2, 12, 16), torch.randn(1, 2, 12, 16), torch.randn(1, 4, 12, 16)
    dq, dk, dv = orc.attention_bwd(q, k, v, g, 0.25, False)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    # group sum: heads 0,1 share kv head 0
    _, dk0, _ = orc.attention_bwd(q[:, :2], k[:, :1], v[:, :1], g[:, :2], 0.25, False)
    assert torch.allclose(dk[:, :1], dk0, atol=1e-5)


def test_backward_matches_autograd():
    torch.manual_seed(1)
    q = torch.randn(1, 2, 9, 8, requires_grad=True)
    k = torch.randn(1, 2, 9, 8, requires_grad=True)
    v = torch.randn(1, 2, 9, 8, requires_grad=True)
    g = torch.randn(1, 2, 9, 8)
    s = (q @ k.transpose(-1, -2)) * 0.3
    s = s.masked_fill(torch.triu(torch.ones(9, 9, dtype=torch.bool), 1), float("-inf"))
    (torch.softmax(s, -1) @ v).backward(g)
    dq, dk, dv = orc.attention_bwd(q.detach(), k.detach(), v.detach(), g, 0.3, True)
    for a, b in ((dq, q.grad), (dk, k.grad), (dv, v.grad)):
        assert torch.allclose(a, b, atol=1e-5)


def test_shifted_causal_mask_is_the_tail_of_the_square_problem():
    """A chunk of the last Nq queries with causal_shift = Nk - Nq sees what those rows see in the
    reference's square causal attention over all Nk positions."""
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 4, 300, 32, generator=g).half()
    k = torch.randn(2, 2, 300, 32, generator=g).half()
    v = torch.randn(2, 2, 300, 32, generator=g).half()
    o_full, lse_full = orc.attention_fwd(q, k, v, 0.2, True)
    for nq in (1, 77, 300):
        o, lse = orc.attention_fwd(q[:, :, -nq:], k, v, 0.2, True, causal_shift=300 - nq)
        assert torch.allclose(o, o_full[:, :, -nq:], atol=1e-6)
        assert torch.allclose(lse, lse_full[:, :, -nq:], atol=1e-6)
    # gradients too: a gradient that is zero outside the last nq rows of the square problem gives the
    # chunk's dQ on those rows and the chunk's dK, dV
    do = torch.randn(2, 4, 300, 32, generator=g).half()
    for nq in (1, 77):
        do_tail = torch.zeros_like(do)
        do_tail[:, :, -nq:] = do[:, :, -nq:]
        dq_f, dk_f, dv_f = orc.attention_bwd(q, k, v, do_tail, 0.2, True)
        dq, dk, dv = orc.attention_bwd(q[:, :, -nq:], k, v, do[:, :, -nq:], 0.2, True, causal_shift=300 - nq)
        assert torch.allclose(dq, dq_f[:, :, -nq:], atol=1e-5)
        assert torch.allclose(dk, dk_f, atol=1e-5) and torch.allclose(dv, dv_f, atol=1e-5)
    # packed form: per-sequence shifts; a sequence with more queries than keys has rows that see nothing
    cu_q, cu_k = torch.tensor([0, 5, 12]), torch.tensor([0, 9, 12])
    qp, kp, vp = torch.randn(12, 2, 8, generator=g), torch.randn(12, 2, 8, generator=g), torch.randn(12, 2, 8, generator=g)
    o, lse = orc.varlen_fwd(qp, kp, vp, cu_q, cu_k, 0.3, True, bottom_right=True)
    o0, _ = orc.attention_fwd(qp[:5].transpose(0, 1)[None], kp[:9].transpose(0, 1)[None], vp[:9].transpose(0, 1)[None],
                              0.3, True, causal_shift=4)
    assert torch.allclose(o[:5], o0[0].transpose(0, 1), atol=1e-6)
    assert torch.isinf(lse[5:9]).all() and (o[5:9] == 0).all()      # 7 queries, 3 keys: the first 4 rows see none
    assert torch.isfinite(lse[9:]).all()


def test_decode_with_a_first_position_equals_the_hook_with_a_padding_mask():
    """decode_fwd(cache_starts=...) against the eager branch of the hook given the additive mask that
    hides each entry's left padding (flash_attn_legacy/integrations.py:80-98)."""
    from flash_attn_legacy.integrations import _eager_attention
    g = torch.Generator().manual_seed(9)
    b, hq, hkv, n, d = 3, 4, 2, 40, 16
    q = torch.randn(b, hq, 1, d, generator=g)
    k, v = torch.randn(b, hkv, n, d, generator=g), torch.randn(b, hkv, n, d, generator=g)
    starts = torch.tensor([0, 13, 39])
    mask = torch.zeros(b, 1, 1, n)
    for i in range(b):
        mask[i, ..., :starts[i]] = float("-inf")
    ref = _eager_attention(q, k, v, mask, 0.3, False)[:, :, 0]
    o, _ = orc.decode_fwd(q[:, :, 0], k.transpose(1, 2), v.transpose(1, 2), torch.full((b,), n), 0.3,
                          cache_starts=starts)
    assert torch.allclose(o, ref, atol=1e-5)


def test_decode_empty_and_full_cache():
    kc, vc, q = torch.randn(2, 8, 1, 16), torch.randn(2, 8, 1, 16), torch.randn(2, 2, 16)
    o, lse = orc.decode_fwd(q, kc, vc, torch.tensor([0, 8]), 0.25)
    assert torch.all(o[0] == 0) and torch.all(torch.isinf(lse[0]))
    ref, _ = orc.attention_fwd(q[1].view(1, 2, 1, 16), kc[1].permute(1, 0, 2)[None], vc[1].permute(1, 0, 2)[None], 0.25)
    assert torch.allclose(o[1], ref.view(2, 16), atol=1e-6)


def test_chunk_against_ragged_caches_is_the_square_problem_per_entry():
    """kvcache_chunk_fwd: for every entry, the chunk's rows equal the last Lq rows of the square causal
    problem over that entry's own positions, whatever the caches hold behind its length."""
    g = torch.Generator().manual_seed(5)
    bsz, hq, hkv, lq, cap, d = 3, 4, 2, 7, 40, 16
    lens = torch.tensor([40, 19, 7], dtype=torch.int32)
    kc = torch.randn(bsz, hkv, cap, d, generator=g)
    vc = torch.randn(bsz, hkv, cap, d, generator=g)
    q = torch.randn(bsz, hq, lq, d, generator=g)
    for b in range(bsz):               # poison what lies behind the lengths
        kc[b, :, int(lens[b]):] = float("nan")
        vc[b, :, int(lens[b]):] = float("inf")
    o, lse = orc.kvcache_chunk_fwd(q, kc, vc, lens, 0.25)
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    for b in range(bsz):
        n = int(lens[b])
        qfull = torch.zeros(1, hq, n, d)
        qfull[:, :, n - lq:] = q[b]
        o_sq, lse_sq = orc.attention_fwd(qfull, kc[b:b + 1, :, :n], vc[b:b + 1, :, :n], 0.25, True)
        assert torch.allclose(o[b], o_sq[0, :, n - lq:], atol=1e-6)
        assert torch.allclose(lse[b], lse_sq[0, :, n - lq:], atol=1e-6)
