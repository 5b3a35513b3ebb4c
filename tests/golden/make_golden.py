"""Generates tests/golden/*.npz by running the REFERENCE's own CPU-runnable code.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/flash-attention-legacy

It imports, unmodified:
  - ref_attention, ref_backward and TestVarlen._ref_varlen from the reference's
    tests/test_flash_attn.py (lines 19-32, 35-58, 293-308), which are
    device-agnostic torch code, and
  - flash_attn_legacy_forward from the reference's flash_attn_legacy/integrations.py,
    whose q_len != kv_len branch (lines 77-98) is pure torch.  The reference package
    imports its CUDA extension at import time; a stub module of that name is put in
    sys.modules so that the import succeeds without a GPU (the stub is never called).

Inputs are seeded N(0,1) fp16; the .npz files hold inputs and the reference's outputs.
"""
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    sys.modules.setdefault("flash_attn_legacy_cuda", types.ModuleType("flash_attn_legacy_cuda"))
    from tests.test_flash_attn import TestVarlen, ref_attention, ref_backward
    from flash_attn_legacy.integrations import flash_attn_legacy_forward

    def randh(gen, *shape):
        return torch.randn(*shape, generator=gen).half()

    # ---- batched forward + backward ---------------------------------------
    cases = [
        # name, B, Hq, Hkv, N, d, causal
        ("mha_d64_causal", 1, 2, 2, 96, 64, True),
        ("gqa_d128_full", 1, 4, 2, 130, 128, False),
        ("mqa_d64_causal_ragged", 2, 4, 1, 77, 64, True),
        ("gqa_d128_causal_300", 1, 4, 1, 300, 128, True),
    ]
    for i, (name, B, Hq, Hkv, N, d, causal) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        q, k, v, do = randh(g, B, Hq, N, d), randh(g, B, Hkv, N, d), randh(g, B, Hkv, N, d), randh(g, B, Hq, N, d)
        scale = 1.0 / math.sqrt(d)
        o = ref_attention(q, k, v, scale, causal)          # fp16, as the reference returns it
        dq, dk, dv = ref_backward(q, k, v, do, scale, causal)
        np.savez_compressed(os.path.join(HERE, f"batched_{name}.npz"),
                            q=q.numpy(), k=k.numpy(), v=v.numpy(), d_out=do.numpy(),
                            o=o.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
                            scale=np.float32(scale), causal=np.bool_(causal))

    # ---- packed forward ------------------------------------------------------
    tv = TestVarlen()
    for i, (name, lens, H, Hkv, d, causal) in enumerate([
        ("varlen_d64_causal", [32, 64, 48], 4, 4, 64, True),
        ("varlen_d128_gqa", [5, 131, 64, 17], 4, 2, 128, False),
    ]):
        g = torch.Generator().manual_seed(200 + i)
        total = sum(lens)
        q, k, v = randh(g, total, H, d), randh(g, total, Hkv, d), randh(g, total, Hkv, d)
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        scale = 1.0 / math.sqrt(d)
        o = tv._ref_varlen(q, k, v, cu, cu, scale, causal)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                            cu_seqlens=cu.numpy(), o=o.numpy(), scale=np.float32(scale),
                            causal=np.bool_(causal))

    # ---- decode: the reference hook's eager branch (q_len = 1) ------------------
    g = torch.Generator().manual_seed(300)
    B, Hq, Hkv, d = 3, 8, 2, 64
    lens = [2, 40, 97]   # kv_len 1 would take the hook's prefill branch (q_len == kv_len)
    S = 128
    kc, vc = randh(g, B, S, Hkv, d), randh(g, B, S, Hkv, d)
    q = randh(g, B, Hq, d)
    scale = 1.0 / math.sqrt(d)
    outs = []
    module = torch.nn.Module()
    for b in range(B):
        n = lens[b]
        # the hook takes [B, H, N, d] tensors; run it in fp32 as a model in float32 would
        kb = kc[b, :n].permute(1, 0, 2).unsqueeze(0).float()
        vb = vc[b, :n].permute(1, 0, 2).unsqueeze(0).float()
        qb = q[b].view(1, Hq, 1, d).float()
        out, _ = flash_attn_legacy_forward(module, qb, kb, vb, None, scaling=scale, is_causal=False)
        outs.append(out.reshape(Hq, d))       # hook returns [B, q_len, H, d]
    np.savez_compressed(os.path.join(HERE, "decode_hook_d64.npz"), q=q.numpy(), k_cache=kc.numpy(),
                        v_cache=vc.numpy(), cache_seqlens=np.array(lens, dtype=np.int32),
                        o=torch.stack(outs).numpy(), scale=np.float32(scale))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of sirCamp/flash-attention-legacy>")
    main(sys.argv[1])
