"""CPU: host-side logic of the Python surface (no kernel launches)."""
import math
import os

import pytest
import torch

from oracle import attention_oracle as orc


@pytest.fixture(scope="module")
def fal():
    import flash_attn_legacy as m
    return m


def test_package_exports_match_the_reference_surface(fal):
    # flash_attn_legacy/__init__.py:46-54 of the reference, plus the decode entry
    for name in ("flash_attention", "flash_attn_varlen_func", "FlashAttention", "FlashMultiHeadAttention",
                 "check_gpu_compatibility", "get_device_info", "register", "flash_attn_with_kvcache"):
        assert name in fal.__all__ and hasattr(fal, name)
    assert fal.__version__ == "0.5.0"


def test_binding_exposes_the_reference_extension_functions():
    import flash_attn_legacy_cuda as ext
    for name in ("forward", "forward_varlen", "backward", "backward_varlen", "decode"):
        assert callable(getattr(ext, name))


def test_head_dims_of_the_reference_are_accepted_without_padding():
    """32 and 96 go to the library as they are (it runs them on its 64 / 128 kernels); the operator
    no longer makes padded copies, and refuses what the reference refuses."""
    from flash_attn_legacy import flash_attn as mod
    assert mod.SUPPORTED_HEAD_DIMS == (32, 64, 96, 128, 256)
    assert not hasattr(mod, "_pad_last")
    with pytest.raises(AssertionError):
        mod.flash_attention(torch.zeros(1, 1, 4, 80, dtype=torch.float16), torch.zeros(1, 1, 4, 80, dtype=torch.float16),
                            torch.zeros(1, 1, 4, 80, dtype=torch.float16))


def test_strided_views_pass_through_and_broadcast_views_are_copied():
    from flash_attn_legacy.flash_attn import _kernel_ready
    x = torch.zeros(2, 50, 4, 64, dtype=torch.float16)
    view = x.transpose(1, 2)                       # [B,H,N,d] view of [B,N,H,d] memory
    assert _kernel_ready(view) is view
    kv = torch.zeros(2, 1, 50, 64, dtype=torch.float16)
    assert _kernel_ready(kv) is kv                 # extent-1 dimensions may have any stride
    wide = kv.expand(2, 4, 50, 64)                 # stride 0 over the heads
    assert wide.stride(1) == 0 and _kernel_ready(wide).stride(1) > 0
    rows = torch.zeros(2, 4, 1, 64, dtype=torch.float16).expand(2, 4, 50, 64)
    assert _kernel_ready(rows).is_contiguous()     # the gradient of a sum over the rows
    assert _kernel_ready(x[..., ::2]).is_contiguous()   # head_dim itself strided


def test_left_padding_is_recognised_and_nothing_else():
    from flash_attn_legacy.integrations import _left_padding_starts
    keep = torch.ones(3, 6, dtype=torch.bool)
    keep[1, :2] = False
    keep[2, :5] = False
    assert _left_padding_starts(keep).tolist() == [0, 2, 5]
    keep[0, 3] = False                      # a hole
    assert _left_padding_starts(keep) is None
    right = torch.ones(2, 6, dtype=torch.bool)
    right[1, 4:] = False                    # right padding
    assert _left_padding_starts(right) is None


def test_operator_asserts_fire_before_any_launch(fal):
    q = torch.zeros(1, 2, 8, 64)
    with pytest.raises(AssertionError):
        fal.flash_attention(q, q, q)                       # not fp16
    with pytest.raises(AssertionError):
        fal.flash_attn_varlen_func(q.half(), q.half(), q.half(), None, None, 8, 8)  # 4-D, not packed
    with pytest.raises(AssertionError):
        fal.FlashMultiHeadAttention(100, num_heads=4)      # head_dim 25
    with pytest.raises(AssertionError):
        fal.FlashMultiHeadAttention(256, num_heads=4, num_kv_heads=3)


def test_binding_refuses_cpu_tensors():
    import flash_attn_legacy_cuda as ext
    q = torch.zeros(1, 2, 8, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        ext.forward(q, q, q, 0.125, False)


def test_causal_flag_resolution_order():
    from flash_attn_legacy.integrations import _resolve_causal

    class M:
        is_causal = False

    assert _resolve_causal(M(), None, 5, {"is_causal": True}) is True      # kwarg wins
    assert _resolve_causal(M(), None, 5, {}) is False                        # then the module's flag
    assert _resolve_causal(object(), None, 5, {}) is True                    # then the heuristic
    assert _resolve_causal(object(), None, 1, {}) is False
    assert _resolve_causal(object(), torch.zeros(1), 5, {}) is False


def test_hook_fallback_branch_matches_the_oracle_on_cpu():
    """On CPU tensors the hook must take the eager branch (the reference's own arithmetic)."""
    from flash_attn_legacy.integrations import flash_attn_legacy_forward
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 8, 1, 32, generator=g)
    k = torch.randn(2, 2, 37, 32, generator=g)
    v = torch.randn(2, 2, 37, 32, generator=g)
    out, weights = flash_attn_legacy_forward(torch.nn.Module(), q, k, v, None, scaling=0.2)
    assert weights is None and out.shape == (2, 1, 8, 32)
    ref, _ = orc.decode_fwd(q[:, :, 0], k.transpose(1, 2), v.transpose(1, 2), torch.tensor([37, 37]), 0.2)
    assert torch.allclose(out[:, 0], ref, atol=1e-5)
    # additive mask and causal chunk: the reference's fallback arithmetic, with the four queries
    # taken as the LAST four of the 37 positions (the reference's triu keeps diagonal=1 there)
    mask = torch.zeros(2, 1, 4, 37)
    mask[..., 1] = float("-inf")
    q4 = torch.randn(2, 8, 4, 32, generator=g)
    out2, _ = flash_attn_legacy_forward(torch.nn.Module(), q4, k, v, mask, scaling=0.2, is_causal=True)
    kk, vv = k.repeat_interleave(4, 1), v.repeat_interleave(4, 1)
    s = q4 @ kk.transpose(-1, -2) * 0.2 + mask + torch.triu(torch.full((4, 37), float("-inf")), 1 + 37 - 4)
    assert torch.allclose(out2, (torch.softmax(s, -1) @ vv).transpose(1, 2), atol=1e-5)


def test_register_is_idempotent_and_patches_validation(fal):
    transformers = pytest.importorskip("transformers")
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS, PreTrainedModel
    assert fal.register() and fal.register()
    assert "flash_attn_legacy" in ALL_ATTENTION_FUNCTIONS.valid_keys()
    check = PreTrainedModel._check_and_adjust_attn_implementation
    assert getattr(check, "_flash_attn_legacy_patched", False)

    class Cfg:
        head_dim = 64

    class Fake:
        config = Cfg()

    assert check(Fake(), "flash_attn_legacy") == "flash_attn_legacy"
    cfg = transformers.LlamaConfig(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                   num_attention_heads=2, num_key_value_heads=1)
    cfg._attn_implementation = "flash_attn_legacy"
    model = transformers.LlamaForCausalLM(cfg)
    assert model.config._attn_implementation == "flash_attn_legacy"
    # a head_dim the kernels do not cover falls back to sdpa, as in the reference
    cfg2 = transformers.LlamaConfig(vocab_size=100, hidden_size=80, intermediate_size=128, num_hidden_layers=1,
                                    num_attention_heads=2, num_key_value_heads=1)
    cfg2._attn_implementation = "flash_attn_legacy"
    model2 = transformers.LlamaForCausalLM(cfg2)
    assert model2.config._attn_implementation == "sdpa"


def test_device_info_needs_cuda(fal):
    if torch.cuda.is_available():
        pytest.skip("covered by the GPU suite")
    with pytest.raises(RuntimeError):
        fal.get_device_info()
    assert fal.check_gpu_compatibility(verbose=False) is False


def test_build_script_keeps_tuning_builds_away_from_the_product_library():
    import importlib.util
    from conftest import PKG
    spec = importlib.util.spec_from_file_location("fal_b200_build_t", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with pytest.raises(RuntimeError):
        mod.build(defines=("FAL_BWD_WAVE_GROUPS=4",))  # a define without --out would replace the product library
    with pytest.raises(RuntimeError):
        mod.build(defines=("FAL_BWD_WAVE_GROUPS=4",), out=mod.LIB_PATH)


def test_padding_mask_reaches_the_hook_and_is_honoured_on_cpu(fal):
    """transformers hands a custom attention function no mask unless a mask format is registered for its
    name; register() does that, and the hook then masks padded keys (here through its eager branch)."""
    transformers = pytest.importorskip("transformers")
    assert fal.register()
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
    assert "flash_attn_legacy" in ALL_MASK_ATTENTION_FUNCTIONS

    def tiny(attn):
        cfg = transformers.LlamaConfig(vocab_size=100, hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                                       num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
        cfg._attn_implementation = attn
        torch.manual_seed(0)
        return transformers.LlamaForCausalLM(cfg).eval()

    ref, model = tiny("eager"), tiny("flash_attn_legacy")
    model.load_state_dict(ref.state_dict())
    assert model.config._attn_implementation == "flash_attn_legacy"
    ids = torch.randint(0, 100, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[1, :5] = 0  # left padding in row 1
    with torch.no_grad():
        a = model(ids, attention_mask=mask).logits
        b = ref(ids, attention_mask=mask).logits
        unmasked = model(ids).logits
    real = mask.bool()
    assert torch.allclose(a[real], b[real], atol=1e-4, rtol=1e-4)
    assert not torch.allclose(a[1, 5:], unmasked[1, 5:], atol=1e-4)  # the mask does change row 1


def test_bench_deals_decode_entries_by_cached_length():
    """bench.py's sharded decode leg: every rank gets 64 / world entries of the same 64 seeded lengths and
    nearly the same number of cached tokens (the ranks are compared by their slowest)."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for world in (2, 4, 8):
        lens, shares = bench.decode_lengths_dealt(world)
        assert len(lens) == 64 and sorted(x for s in shares for x in s) == sorted(lens)
        assert all(len(s) == 64 // world for s in shares)
        totals = [sum(s) for s in shares]
        assert max(totals) <= 1.05 * min(totals)
        assert bench.decode_lengths_dealt(world)[0] == lens      # seeded: the same on every rank
