"""Prints where the forward kernel's cycles go, from a library built with its cycle counters.

    python flash-attention-legacy_b200/build.py --define FAL_FWD_TIMING --out /tmp/libfal_timing.so
    FAL_B200_LIB=/tmp/libfal_timing.so python flash-attention-legacy_b200/csrc/forward_cycles.py
    FAL_B200_LIB=/tmp/libfal_timing.so FAL_FWD_PAIR=1 python flash-attention-legacy_b200/csrc/forward_cycles.py

Shape: B4 Hq32 Hkv8 N4096 d128 (the bench workload), both mask settings.  Figures are cycles per
128x128 tile-step (issuer) or per step of one tile (softmax warp 0 of each tile), clock reads included.
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import flash_attn_legacy_cuda as ext  # noqa: E402

which = "fwd_pair" if os.environ.get("FAL_FWD_PAIR") == "1" else "fwd"
if ext.debug_cycles(which) is None:
    sys.exit("this library was built without -DFAL_FWD_TIMING")
B, Hq, Hkv, N, d = 4, 32, 8, 4096, 128
torch.manual_seed(0)
q = torch.randn(B, Hq, N, d, device="cuda").half()
k = torch.randn(B, Hkv, N, d, device="cuda").half()
v = torch.randn(B, Hkv, N, d, device="cuda").half()
scale = 1 / math.sqrt(d)
for causal in (False, True):
    for _ in range(3):
        ext.forward(q, k, v, scale, causal)
    torch.cuda.synchronize()
    ext.debug_cycles(which)
    ext.forward(q, k, v, scale, causal)
    torch.cuda.synchronize()
    c = ext.debug_cycles(which)
    steps, total = max(c[5], 1), c[4]
    print(f"causal={causal}: issuer {total / steps:.0f} cycles per tile-step over {steps} tile-steps")
    issuer = [(0, "wait P first half"), (1, "wait V (pair kernel: commits)"), (2, "wait P second half"),
              (3, "wait K"), (23, "issue P V first half (4 MMAs)"), (24, "issue P V second half (4 MMAs)"),
              (25, "issue Q K^T (8 MMAs)")]
    for i, name in issuer:
        print(f"  issuer  {name:34s} {c[i] / steps:7.0f}")
    sm_steps = max(c[16], 1)
    print(f"  softmax warp: {c[14] / sm_steps:.0f} cycles per step over {sm_steps} steps")
    softmax = [(15, "loop overhead"), (8, "wait for S"), (9, "S to registers"), (10, "mask + row maximum"),
               (11, "rescale decision"), (12, "P first half"), (13, "P second half")]
    for i, name in softmax:
        print(f"  softmax {name:34s} {c[i] / sm_steps:7.0f}")
