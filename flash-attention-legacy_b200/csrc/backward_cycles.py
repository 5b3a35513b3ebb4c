"""Prints where the backward kernel's cycles go, from a library built with its cycle counters.

    python flash-attention-legacy_b200/build.py --define FAL_BWD_TIMING --out /tmp/libfal_timing.so
    FAL_B200_LIB=/tmp/libfal_timing.so python flash-attention-legacy_b200/csrc/backward_cycles.py

Shape: B4 Hq32 Hkv8 N4096 d128 causal (the bench workload).  Figures are cycles per 128x128
(key tile, query tile) pair, summed over CTAs and divided by the number of pairs; clock reads included.
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import flash_attn_legacy_cuda as ext  # noqa: E402

if ext.debug_cycles("bwd") is None:
    sys.exit("this library was built without -DFAL_BWD_TIMING")
B, Hq, Hkv, N, d = 4, 32, 8, 4096, 128
torch.manual_seed(0)
q = torch.randn(B, Hq, N, d, device="cuda").half()
k = torch.randn(B, Hkv, N, d, device="cuda").half()
v = torch.randn(B, Hkv, N, d, device="cuda").half()
do = torch.randn(B, Hq, N, d, device="cuda").half()
scale = 1 / math.sqrt(d)
o, lse = ext.forward(q, k, v, scale, True)
for _ in range(2):
    ext.backward(do, q, k, v, o, lse, scale, True)
torch.cuda.synchronize()
ext.debug_cycles("bwd")
ext.backward(do, q, k, v, o, lse, scale, True)
torch.cuda.synchronize()
c = ext.debug_cycles("bwd")
pairs, ctas, total = max(c[13], 1), c[14], c[12]
print(f"ctas={ctas} pairs={pairs} cycles per pair={total / pairs:.0f}")
waits = ["producer: stage empty", "issuer: dO full", "issuer: P ready", "issuer: Q full", "issuer: dQ free",
         "issuer: dS ready", "compute: statistics full", "compute: S ready", "compute: dP ready",
         "compute: dS buffer free", "write-back: dQ ready", "write-back: reduce section"]
for i, name in enumerate(waits):
    print(f"  wait  {name:32s} {c[i] / pairs:7.0f}")
phases = ["compute: P load + wait", "compute: P exponentials", "compute: P store + wait", "compute: dS load + wait",
          "compute: dS until buffer free", "producer: dO empty wait", "compute: P phase, waits inside included",
          "compute: dS phase, buffer wait included"]
for i, name in zip(range(16, 24), phases):
    print(f"  phase {name:40s} {c[i] / pairs:7.0f}")
