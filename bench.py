"""Headline benchmark: causal GQA attention forward + backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (one "step" = one forward + one backward over one batch of synthetic input):
    B=4, Hq=32, Hkv=8, N=4096, d=128, causal, fp16, scale 1/sqrt(128); q, k, v, dO iid N(0,1).
Algorithmic work per step = 3.5 * (4*B*Hq*N*N*d / 2) = 1.924e12 FLOP (forward 2 GEMMs,
backward 5; the causal half is counted once; recompute and softmax are not counted).

Prints ONE JSON line.  `value` is whole-job TFLOP/s with inputs resident in HBM (kernel
path through the C-ABI with preallocated outputs); `e2e` is the same metric through the
public autograd API from pinned HOST buffers, host<->device copies inside the timed
region.  With --gpus N each rank (one process per GPU) runs the same workload on its own
shard of independent (batch, head-group) units -- no collective on the data path -- and
the time is the maximum over ranks.

With --gpus N > 1 the line also carries `extra.sharded`: one timed leg per partitioning of the other
sharded configurations on the same ranks (strong scaling: the total work is that of one GPU's
problem) -- the headline workload with its 32 (batch, KV-head group) units dealt to the ranks, the
packed workload with its heads dealt, the decode workload with its batch entries dealt, and the
131072-token sequence in the zigzag ring -- each with its own one-GPU time taken in the same run,
the efficiency against it, the device status word and a sampled error against the CPU oracle
(rank 0, outside every timed region; the oracle is only ever the checker).

--impl reference times the reference's CPU math path (the fp32 naive attention its
tests use, restated in oracle/attention_oracle.py) on the host cores, on a bounded
sample of the same workload.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "flash-attention-legacy_b200"))

WORKLOAD = dict(B=4, Hq=32, Hkv=8, N=4096, d=128, causal=True)
WORKLOAD_NAME = "gqa_fwd_bwd_B4_Hq32_Hkv8_N4096_d128_causal_fp16"
METRIC = "attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def step_flops(w=WORKLOAD):
    fwd = 4.0 * w["B"] * w["Hq"] * w["N"] * w["N"] * w["d"] * (0.5 if w["causal"] else 1.0)
    return fwd, 2.5 * fwd


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return {"bf16_tflops": m.get("bf16_tflops"), "bf16_tflops_sustained": m.get("bf16_tflops_sustained"),
                "hbm_gbs": m.get("hbm_gbs"), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


KERNEL_SOURCES = ("fal_bwd.cu", "sm100_ptx.cuh", "fal_common.h")


def kernel_source_hash():
    """sha256 over the files the backward kernel is compiled from (what an ncu capture belongs to)."""
    import hashlib
    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        with open(os.path.join(ROOT, "flash-attention-legacy_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def recorded_traffic():
    """DRAM bytes per launch of the backward kernel on the bench workload, from the tracked record of
    the last ncu capture -- or None with the reason when that record belongs to other kernel sources
    or another workload (a stale figure must not ride along with a new build)."""
    path = os.path.join(ROOT, "profiles", "bwd_kernel_config2.traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)
    except (OSError, ValueError):
        return None, "no capture record"
    if rec.get("workload") != WORKLOAD_NAME:
        return None, "the capture record is for another workload"
    if rec.get("kernel_source_sha256") != kernel_source_hash():
        return None, "kernel sources changed since the capture (%s)" % rec.get("captured_at_commit", "?")
    return float(rec["dram_bytes_read"]) + float(rec["dram_bytes_write"]), "ncu capture at commit %s" % rec.get(
        "captured_at_commit", "?")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs.

    Only samples whose timestamp falls inside [mark_begin(), mark_end()] are used, so that idle
    clocks before and after the timed region do not leak into the median.
    """

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    @staticmethod
    def _parse_ts(text):
        import datetime
        try:
            return datetime.datetime.strptime(text.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside, everything, mx, reasons = [], [], [], set()
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clk, clk_max = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            ts = self._parse_ts(parts[0])
            in_window = (ts is not None and self.t_begin is not None and self.t_end is not None
                         and self.t_begin - 0.02 <= ts <= self.t_end + 0.02)
            everything.append(clk)
            mx.append(clk_max)
            if in_window:
                inside.append(clk)
                for name, val in zip(names, parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        used = sorted(inside if inside else everything)
        med = used[len(used) // 2] if used else None
        return {"sm_mhz": med, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples_in_timed_region": len(inside), "samples_total": len(everything)}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    torch.cuda.set_device(0)
    return 0, 1, 0, None


def cpu_baseline_sample(num_slices, min_seconds=0.0):
    """Times the oracle's forward + backward on (batch, kv-head-group) slices of the workload: at least
    `num_slices` of them, and as many more as it takes to fill `min_seconds` (32 at most -- the step).

    One slice = 1 batch entry x 4 query heads x 1 KV head x N=4096 x d=128 (1/32 of a step).
    Returns (tflops, seconds, threads, slices).
    """
    sys.path.insert(0, ROOT)
    from oracle import attention_oracle as orc
    w = WORKLOAD
    group = w["Hq"] // w["Hkv"]
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, group, w["N"], w["d"], generator=g).half()
    k = torch.randn(1, 1, w["N"], w["d"], generator=g).half()
    v = torch.randn(1, 1, w["N"], w["d"], generator=g).half()
    do = torch.randn(1, group, w["N"], w["d"], generator=g).half()
    scale = 1.0 / math.sqrt(w["d"])
    fwd, bwd = step_flops()
    slice_flops = (fwd + bwd) / (w["B"] * w["Hkv"])
    t0 = time.perf_counter()
    done = 0
    while done < num_slices or (time.perf_counter() - t0 < min_seconds and done < w["B"] * w["Hkv"]):
        orc.attention_fwd(q, k, v, scale, w["causal"])
        orc.attention_bwd(q, k, v, do, scale, w["causal"])
        done += 1
    dt = time.perf_counter() - t0
    return slice_flops * done / dt / 1e12, dt, torch.get_num_threads(), done


def run_reference(args):
    """Reference arm: the reference's fp32 CPU math path, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    slices_per_step = 1
    # All the host cores this process may use (torchrun exports OMP_NUM_THREADS=1 by default).
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    for _ in range(min(args.warmup, 1)):
        cpu_baseline_sample(1)
    t_total, tf_list = 0.0, []
    for _ in range(args.steps):
        tf, dt, threads, _ = cpu_baseline_sample(slices_per_step)
        tf_list.append(tf)
        t_total += dt
    value = sum(tf_list) / len(tf_list)
    sample = (f"{slices_per_step} of 32 (batch, kv-head-group) slices per step: 4 query heads x 1 KV head, "
              "N=4096, d=128, fp32 forward + closed-form backward")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD_NAME, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_decode_extra(ext, peaks, steps=256, batch=64, seed=3, graph=False, check=False, lens_init=None):
    """Secondary metric: KV-cache split-K decode with appends, B=64 Hq=32 Hkv=8 d=128, cache 32768.

    graph=True captures one step (split-K with append, combine, the length increment) in a CUDA graph
    and replays it `steps` times: a small per-GPU batch is otherwise bound by the host's launch path,
    not by the kernels.  Every replay appends the same new token (at a new position) and uses the same
    query; the kernels and the bytes they move are those of the eager loop.
    lens_init: the entries' starting lengths (a rank's share of a batch dealt by length); else seeded."""
    B, Hq, Hkv, S, d = (batch if lens_init is None else len(lens_init)), 32, 8, 32768, 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    kc = torch.randn(B, S, Hkv, d, device="cuda", dtype=torch.float16, generator=g)
    vc = torch.randn(B, S, Hkv, d, device="cuda", dtype=torch.float16, generator=g)
    lens0 = torch.randint(1024, S - steps + 1, (B,), device="cuda", generator=g).to(torch.int32)
    if lens_init is not None:
        lens0 = torch.as_tensor(lens_init, dtype=torch.int32).cuda()
    q = torch.randn(steps, B, Hq, d, device="cuda", dtype=torch.float16, generator=g)
    kn = torch.randn(steps, B, Hkv, d, device="cuda", dtype=torch.float16, generator=g)
    vn = torch.randn(steps, B, Hkv, d, device="cuda", dtype=torch.float16, generator=g)
    out = torch.empty(B, Hq, d, device="cuda", dtype=torch.float16)
    scale = 1.0 / math.sqrt(d)
    # Warm-up runs the WHOLE step, the length increment included: the first use of a framework
    # kernel in a process loads its module (about 15 ms once -- inside a 256-step timed loop that was
    # 60 us per step on an 8-entry batch).  The appended rows are overwritten by the timed steps.
    lens = lens0.clone()
    for i in range(min(8, steps)):
        ext.decode(q[i], kc, vc, lens, scale, kn[i], vn[i], out=out)
        lens += 1
    torch.cuda.synchronize()
    lens = lens0.clone()
    ext.profile_read(ext.KERNEL_DECODE_SPLITK)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            ext.decode(q[0], kc, vc, lens, scale, kn[0], vn[0], out=out)
            lens += 1
        lens.copy_(lens0)
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            cg.replay()
        e1.record()
    else:
        e0.record()
        for i in range(steps):
            ext.decode(q[i], kc, vc, lens, scale, kn[i], vn[i], out=out)
            lens += 1
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    k_ms, k_n = ext.profile_read(ext.KERNEL_DECODE_SPLITK)
    mean_len = lens0.float().mean().item() + (steps + 1) / 2.0
    kv_bytes = mean_len * B * Hkv * d * 2 * 2  # K and V, fp16, read once per KV head
    res = {"workload": f"decode_B{B}_Hq32_Hkv8_d128_cache32768_{steps}steps_with_append",
           "ms_per_step": ms, "kv_bytes_per_step": kv_bytes, "kv_gbs": kv_bytes / ms / 1e6,
           "frac_of_hbm_peak": kv_bytes / ms / 1e6 / peaks["hbm_gbs"], "hbm_peak_gbs": peaks["hbm_gbs"],
           "launches_per_step": 2, "launch_path": "cuda graph replay" if graph else "eager"}
    if k_n:
        res["splitk_kernel_ms"] = k_ms / k_n
        res["splitk_kernel_gbs"] = kv_bytes / (k_ms / k_n) / 1e6
    if check and not graph:
        # the last step's output of two entries against the CPU oracle (the checker, never the product)
        orc = _oracle()
        idx = torch.tensor([0, B - 1], device="cuda")
        o_ref, _ = orc.decode_fwd(q[steps - 1][idx].cpu(), kc[idx].cpu(), vc[idx].cpu(), lens[idx].cpu(), scale)
        res["check"] = {"checked": "entries 0 and %d after the last step" % (B - 1),
                        "o": orc.rel_max_err(out[idx], o_ref)}
    del kc, vc
    torch.cuda.empty_cache()
    return res


def decode_lengths_dealt(world, steps=256, batch=64, capacity=32768, seed=3):
    """The decode workload's starting lengths (seeded, the same on every rank) and their deal to the ranks:
    sorted by length and handed out back and forth, so every rank gets batch / world entries and nearly the
    same number of cached tokens (the ranks' step times are compared by their maximum).
    -> (all lengths, [the lengths of rank 0, of rank 1, ...])."""
    lens = torch.randint(1024, capacity - steps + 1, (batch,), generator=torch.Generator().manual_seed(seed)).tolist()
    order = sorted(range(batch), key=lambda i: -lens[i])
    shares = [[] for _ in range(world)]
    for pos, i in enumerate(order):
        rnd, slot = divmod(pos, world)
        shares[slot if rnd % 2 == 0 else world - 1 - slot].append(lens[i])
    return lens, shares


def _max_over_ranks(dist, dev, x):
    if dist is None:
        return x
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def run_varlen(args, rank, world, local, dist, ext):
    """Secondary metric: 16 packed causal sequences of 64..4096 tokens (seeded), H=16, d=128, forward +
    backward.  The 16 heads are dealt to the ranks (every rank sees the same length mix); no collective."""
    H, d, num_seqs = 16, 128, 16
    if H % world != 0:
        raise SystemExit("the varlen workload shards 16 heads: use 1, 2, 4, 8 or 16 ranks")
    h_local = H // world
    dev = torch.device("cuda", local)
    lens = torch.randint(64, 4097, (num_seqs,), generator=torch.Generator().manual_seed(2))
    cu = torch.zeros(num_seqs + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    total, max_len = int(cu[-1]), int(lens.max())
    cu = cu.to(dev)
    gen = torch.Generator(device="cuda").manual_seed(20 + rank)
    q, k, v, do = (torch.randn(total, h_local, d, device=dev, generator=gen).half() for _ in range(4))
    scale = 1.0 / math.sqrt(d)

    def step():
        o, lse = ext.forward_varlen(q, k, v, cu, cu, max_len, max_len, scale, True)
        return ext.backward_varlen(do, q, k, v, o, lse, cu, cu, max_len, max_len, scale, True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = _max_over_ranks(dist, dev, e0.elapsed_time(e1) / args.steps)
    flops = 3.5 * 2.0 * H * d * float((lens.double() ** 2).sum())  # causal half counted once
    status = ext.device_status()
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"varlen_16seqs_64to4096_{total}tokens_H16_d128_causal_fwd_bwd",
                       "parallelism": f"{h_local} of 16 heads per rank, no collective"},
            "device_status": status}))
    if dist is not None:
        dist.destroy_process_group()


def run_shapes(args, ext):
    """Kernel timing on stated shapes, one JSON line each (one GPU).  A shape is
    `pass:B,Hq,Hkv,Nq,Nk,d[:noncausal]` with pass = fwd, bwd (backward incl. its pre- and post-pass; Nq = Nk)
    chunk (forward of the last Nq positions against Nk keys, causal mask aligned to the end of the keys)
    or kvchunk (chunk against caches of capacity Nk filled to a different length per entry, seeded lengths
    between Nq and Nk).  FLOPs: 4*Hq*d per visible (query, key) pair forward, 2.5x that backward."""
    for spec in args.shape:
        parts = spec.split(":")
        kind = parts[0]
        B, Hq, Hkv, Nq, Nk, d = (int(x) for x in parts[1].split(","))
        causal = not (len(parts) > 2 and parts[2] == "noncausal")
        gen = torch.Generator(device="cuda").manual_seed(7)
        q = torch.randn(B, Hq, Nq, d, device="cuda", generator=gen).half()
        k = torch.randn(B, Hkv, Nk, d, device="cuda", generator=gen).half()
        v = torch.randn(B, Hkv, Nk, d, device="cuda", generator=gen).half()
        do = torch.randn(B, Hq, Nq, d, device="cuda", generator=gen).half()
        scale = 1.0 / math.sqrt(d)
        if kind == "chunk":
            pairs = Nq * (Nk - Nq) + Nq * (Nq + 1) / 2.0
            fn = lambda: ext.forward_rect(q, k, v, scale, True, bottom_right=True)
            mult = 1.0
        elif kind == "kvchunk":
            lens = torch.randint(Nq, Nk + 1, (B,), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
            pairs = float(sum(Nq * (int(n) - Nq) + Nq * (Nq + 1) / 2.0 for n in lens)) / B  # per batch entry
            lens_dev = lens.cuda()
            fn = lambda: ext.forward_kvcache(q, k, v, lens_dev, scale, True)
            mult = 1.0
        else:
            if Nq != Nk:
                raise SystemExit("fwd / bwd shapes need Nq == Nk")
            pairs = Nq * (Nq + 1) / 2.0 if causal else float(Nq) * Nk
            if kind == "fwd":
                fn = lambda: ext.forward(q, k, v, scale, causal)
                mult = 1.0
            elif kind == "bwd":
                o, lse = ext.forward(q, k, v, scale, causal)
                fn = lambda: ext.backward(do, q, k, v, o, lse, scale, causal)
                mult = 2.5
            else:
                raise SystemExit(f"unknown pass {kind!r}: fwd, bwd, chunk or kvchunk")
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        kind_id = ext.KERNEL_BWD if kind == "bwd" else ext.KERNEL_FWD
        ext.profile_enable(True)
        ext.profile_read(kind_id)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        k_ms, k_n = ext.profile_read(kind_id)
        ext.profile_enable(False)
        ms = e0.elapsed_time(e1) / args.steps
        flops = mult * 4.0 * B * Hq * d * pairs
        # ms_per_step: back-to-back calls from Python (a small problem is bound by the host there);
        # main_kernel_ms: the library's event pair around the main kernel alone
        print(json.dumps({"metric": "attn_kernel_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT,
                          "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                          "main_kernel_ms": k_ms / k_n if k_n else None,
                          "main_kernel_tflops": flops / (k_ms / k_n * 1e-3) / 1e12 if k_n else None,
                          "dtype": "f16", "data": "synthetic",
                          "config": {"workload": spec, "pass": kind, "causal": causal,
                                     "l2_policy": "back-to-back launches on the same tensors"},
                          "device_status": ext.device_status()}))


def run_decode(args, rank, world, local, dist, ext):
    """Secondary metric: the KV-cache decode of run_decode_extra with its 64 batch entries dealt to
    the ranks (each rank holds its entries' caches); no collective.  Metric: KV bytes streamed per second."""
    if 64 % world != 0:
        raise SystemExit("the decode workload shards 64 batch entries: use a power-of-two rank count")
    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    if dist is not None:
        dist.barrier()
    shard = args.decode_batch if (world == 1 and args.decode_batch > 0) else 64 // world
    share = decode_lengths_dealt(world)[1][rank] if world > 1 else None
    res = run_decode_extra(ext, peaks, steps=256, batch=shard, seed=3 + rank, graph=args.decode_graph, lens_init=share)
    ms = _max_over_ranks(dist, dev, res["ms_per_step"])
    total_bytes = res["kv_bytes_per_step"]
    if dist is not None:
        t = torch.tensor([total_bytes], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        total_bytes = t.item()
    status = ext.device_status()
    if rank == 0:
        gbs = total_bytes / ms / 1e6
        print(json.dumps({
            "metric": "decode_kv_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": 256,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "decode_B64_Hq32_Hkv8_d128_cache32768_256steps_with_append",
                       "parallelism": f"{shard} of 64 batch entries per rank, dealt by cached length, no collective",
                       "launch_path": res["launch_path"]},
            "frac_of_hbm_peak_per_gpu": gbs / world / peaks["hbm_gbs"], "hbm_peak_gbs": peaks["hbm_gbs"],
            "device_status": status}))
    if dist is not None:
        dist.destroy_process_group()


def run_long_context(args, rank, world, local, dist, ext):
    """Secondary metric: one 131072-token causal sequence, forward + backward, context parallel.

    With one rank the kernels run on the whole sequence; with more, K/V shards travel the ring (NCCL
    point-to-point) while the kernels work on the shard already present.  Layout "zigzag" (default):
    the sequence is cut into 2G chunks, rank r holds chunks r and 2G-1-r, every rank does the same
    work in every ring step.  Layout "contiguous": rank r holds rows [r*N/G, (r+1)*N/G) and has r+1
    shard pairs to do under the causal mask, so the last rank sets the time.
    """
    from flash_attn_legacy import distributed as fd
    B, Hq, Hkv, N, d = 1, 32, 8, 131072, 128
    scale = 1.0 / math.sqrt(d)
    dev = torch.device("cuda", local)
    lo, hi = fd.shard_range(N, world, rank)
    n_local = hi - lo
    gen = torch.Generator(device="cuda").manual_seed(4 + rank)
    q = torch.randn(B, Hq, n_local, d, device=dev, generator=gen).half()
    k = torch.randn(B, Hkv, n_local, d, device=dev, generator=gen).half()
    v = torch.randn(B, Hkv, n_local, d, device=dev, generator=gen).half()
    do = torch.randn(B, Hq, n_local, d, device=dev, generator=gen).half()

    def step():
        if world == 1:
            o, lse = ext.forward(q, k, v, scale, True)
            return ext.backward(do, q, k, v, o, lse, scale, True)
        o, lse = fd.ring_attention_forward(q, k, v, scale, True, layout=args.ring_layout)
        return fd.ring_attention_backward(do, q, k, v, o, lse, scale, True, layout=args.ring_layout)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    barrier()
    steps = max(1, min(args.steps, 5))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    flops = 3.5 * 4.0 * B * Hq * N * N * d * 0.5
    status = ext.device_status()
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": steps, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "long_context_B1_Hq32_Hkv8_N131072_d128_causal_fwd_bwd",
                       "parallelism": f"{args.ring_layout} sequence shards over {world} rank(s), ring K/V exchange"
                                      if world > 1 else "one rank, whole sequence"},
            "device_status": status}))
    if dist is not None:
        dist.destroy_process_group()

# ---------------------------------------------------------------------------------------------
# Sharded legs (--gpus N > 1): strong scaling of the other partitionings, on the same ranks
# ---------------------------------------------------------------------------------------------
def _time_steps(fn, steps, warmup, dist, dev):
    """Device time per step of fn(): warm-up, barrier + sync on both sides, max over ranks."""
    for _ in range(warmup):
        fn()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    return _max_over_ranks(dist, dev, e0.elapsed_time(e1) / steps)


def _oracle():
    sys.path.insert(0, ROOT)
    from oracle import attention_oracle as orc
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))  # torchrun exports OMP_NUM_THREADS=1
    return orc


def leg_units_split(args, rank, world, dev, dist, ext, full_ms):
    """The headline workload's 32 (batch, KV-head group) units dealt to the ranks: every rank gets all
    four batch entries and 8 / N KV heads with their query heads."""
    w = WORKLOAD
    hkv = w["Hkv"] // world
    hq = hkv * (w["Hq"] // w["Hkv"])
    B, N, d = w["B"], w["N"], w["d"]
    scale = 1.0 / math.sqrt(d)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    q, do = (torch.randn(B, hq, N, d, device=dev, generator=gen).half() for _ in range(2))
    k, v = (torch.randn(B, hkv, N, d, device=dev, generator=gen).half() for _ in range(2))
    o = torch.empty_like(q)
    lse = torch.empty(B, hq, N, device=dev, dtype=torch.float32)
    grads = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    ws = torch.empty(ext.backward_workspace_bytes(B, hq, N, d), dtype=torch.uint8, device=dev)

    def step():
        ext.forward(q, k, v, scale, True, out=o, lse=lse)
        ext.backward(do, q, k, v, o, lse, scale, True, out=grads, workspace=ws)

    ms = _time_steps(step, args.steps, args.warmup, dist, dev)
    fwd, bwd = step_flops()
    res = {"workload": WORKLOAD_NAME, "parallelism": f"{B * hkv} of 32 (batch, KV-head group) units per rank, no collective",
           "ms_per_step": ms, "value": (fwd + bwd) / (ms * 1e-3) / 1e12, "unit": UNIT,
           "one_gpu_ms_per_step": full_ms, "efficiency_vs_one_gpu": full_ms / (world * ms)}
    if rank == 0:
        orc = _oracle()
        sl = slice(0, 4)
        qs, ks, vs, gs = q[1:2, sl].cpu(), k[1:2, :1].cpu(), v[1:2, :1].cpu(), do[1:2, sl].cpu()
        o_ref, lse_ref = orc.attention_fwd_blocked(qs, ks, vs, scale, True)
        ref = orc.attention_bwd_blocked(qs, ks, vs, gs, scale, True)
        res["sampled_error_vs_oracle"] = {
            "checked": "one (batch, KV-head group) unit of rank 0 in full",
            "o": orc.rel_max_err(o[1:2, sl], o_ref), "lse_abs": orc.abs_max_err(lse[1:2, sl], lse_ref),
            "dq": orc.rel_max_err(grads[0][1:2, sl], ref[0]), "dk": orc.rel_max_err(grads[1][1:2, :1], ref[1]),
            "dv": orc.rel_max_err(grads[2][1:2, :1], ref[2])}
    res["device_status"] = ext.device_status()
    return res


def leg_varlen_split(args, rank, world, dev, dist, ext):
    """16 packed causal sequences of 64..4096 tokens (seed 2), H=16, d=128, forward + backward: the heads
    dealt to the ranks.  The one-GPU time (all 16 heads) is taken on every rank in the same run."""
    H, d, num_seqs = 16, 128, 16
    lens = torch.randint(64, 4097, (num_seqs,), generator=torch.Generator().manual_seed(2))
    cu_host = torch.zeros(num_seqs + 1, dtype=torch.int32)
    cu_host[1:] = torch.cumsum(lens, 0)
    total, max_len = int(cu_host[-1]), int(lens.max())
    cu = cu_host.to(dev)
    scale = 1.0 / math.sqrt(d)
    flops = 3.5 * 2.0 * H * d * float((lens.double() ** 2).sum())
    out = {}
    for label, heads in (("one_gpu", H), ("shard", H // world)):
        gen = torch.Generator(device="cuda").manual_seed(200 + rank)
        q, k, v, do = (torch.randn(total, heads, d, device=dev, generator=gen).half() for _ in range(4))
        keep = {}

        def step():
            o, lse = ext.forward_varlen(q, k, v, cu, cu, max_len, max_len, scale, True)
            keep["o"], keep["g"] = o, ext.backward_varlen(do, q, k, v, o, lse, cu, cu, max_len, max_len, scale, True)

        out[label] = _time_steps(step, args.steps, args.warmup, dist, dev)
        if label == "shard":
            shard = (q, k, v, do, keep["o"], keep["g"])
    ms = out["shard"]
    res = {"workload": f"varlen_16seqs_64to4096_{total}tokens_H16_d128_causal_fwd_bwd",
           "parallelism": f"{H // world} of 16 heads per rank, no collective", "ms_per_step": ms,
           "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "one_gpu_ms_per_step": out["one_gpu"],
           "efficiency_vs_one_gpu": out["one_gpu"] / (world * ms)}
    if rank == 0:
        orc = _oracle()
        q, k, v, do, o, g = shard
        order = torch.argsort(lens)[:6].tolist()   # the six shortest sequences of head 0
        worst = {"o": 0.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
        for s_i in order:
            a, e = int(cu_host[s_i]), int(cu_host[s_i + 1])
            pick = lambda t: t[a:e, :1].permute(1, 0, 2).unsqueeze(0).cpu()
            o_ref, _ = orc.attention_fwd(pick(q), pick(k), pick(v), scale, True)
            ref = orc.attention_bwd(pick(q), pick(k), pick(v), pick(do), scale, True)
            worst["o"] = max(worst["o"], orc.rel_max_err(pick(o), o_ref))
            for name, got, want in zip(("dq", "dk", "dv"), g, ref):
                worst[name] = max(worst[name], orc.rel_max_err(pick(got), want))
        res["sampled_error_vs_oracle"] = dict(worst, checked="head 0 of rank 0 on the six shortest sequences")
    res["device_status"] = ext.device_status()
    return res


def leg_decode_split(args, rank, world, dev, dist, ext, peaks):
    """The decode workload (batch 64, cache 32768, 256 steps with appends): the batch entries dealt to the
    ranks.  The one-GPU time (all 64 entries) is taken on every rank in the same run."""
    all_lens, shares = decode_lengths_dealt(world)
    full = run_decode_extra(ext, peaks, steps=256, seed=300 + rank, lens_init=all_lens)
    full_ms = _max_over_ranks(dist, dev, full["ms_per_step"])
    shard_n = 64 // world
    part = run_decode_extra(ext, peaks, steps=256, seed=300 + rank, check=(rank == 0), lens_init=shares[rank])
    ms = _max_over_ranks(dist, dev, part["ms_per_step"])
    total_bytes = part["kv_bytes_per_step"]
    if dist is not None:
        t = torch.tensor([total_bytes], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        total_bytes = t.item()
    res = {"workload": "decode_B64_Hq32_Hkv8_d128_cache32768_256steps_with_append",
           "parallelism": f"{shard_n} of 64 batch entries per rank, dealt by cached length (the same 64 lengths as the "
                          "one-GPU run), no collective", "launch_path": "eager, two launches per step",
           "ms_per_step": ms, "value": total_bytes / ms / 1e6, "unit": "GB/s",
           "frac_of_hbm_peak_per_gpu": total_bytes / ms / 1e6 / world / peaks["hbm_gbs"],
           "one_gpu_ms_per_step": full_ms, "efficiency_vs_one_gpu": full_ms / (world * ms)}
    if "check" in part:
        res["sampled_error_vs_oracle"] = part["check"]
    res["device_status"] = ext.device_status()
    return res


def leg_ring(args, rank, world, local, dev, dist, ext):
    """One 131072-token causal sequence, forward + backward, zigzag rows over the ranks with the ring K/V
    exchange.  The one-GPU time (the whole sequence on one GPU) is taken on every rank in the same run."""
    from flash_attn_legacy import distributed as fd
    B, Hq, Hkv, N, d = 1, 32, 8, 131072, 128
    scale = 1.0 / math.sqrt(d)
    flops = 3.5 * 4.0 * B * Hq * N * N * d * 0.5

    def local_inputs(r, rows):
        gen = torch.Generator(device="cuda").manual_seed(400 + r)
        return [torch.randn(B, h, rows, d, device=dev, generator=gen).half() for h in (Hq, Hkv, Hkv, Hq)]

    q, k, v, do = local_inputs(1000 + rank, N)

    def whole():
        o, lse = ext.forward(q, k, v, scale, True)
        ext.backward(do, q, k, v, o, lse, scale, True)

    one_gpu_ms = _time_steps(whole, 2, 1, dist, dev)
    del q, k, v, do
    torch.cuda.empty_cache()
    rows = N // world
    q, k, v, do = local_inputs(rank, rows)
    keep = {}

    def step():
        o, lse = fd.ring_attention_forward(q, k, v, scale, True, layout="zigzag", check_shards=False)
        keep["o"], keep["lse"] = o, lse
        keep["g"] = fd.ring_attention_backward(do, q, k, v, o, lse, scale, True, layout="zigzag", check_shards=False)

    ms = _time_steps(step, 3, 1, dist, dev)
    res = {"workload": "long_context_B1_Hq32_Hkv8_N131072_d128_causal_fwd_bwd",
           "parallelism": f"zigzag sequence shards over {world} ranks, ring K/V exchange (NCCL point-to-point)",
           "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT,
           "one_gpu_ms_per_step": one_gpu_ms, "efficiency_vs_one_gpu": one_gpu_ms / (world * ms)}
    if rank == 0:
        # Rank 0 holds the first and the LAST chunk of the sequence: its last 256 local rows are the last
        # 256 rows of the whole problem and see every key.  Every rank's K/V of one KV head is regenerated
        # here from its seed and put in sequence order.
        orc = _oracle()
        h = 3
        c = rows // 2
        kf = torch.empty(1, 1, N, d)
        vf = torch.empty(1, 1, N, d)
        for r in range(world):
            _, kr, vr, _ = local_inputs(r, rows)
            (a0, a1), (b0, b1) = fd.zigzag_rows(N, world, r)
            kf[:, :, a0:a1], kf[:, :, b0:b1] = kr[:, h:h + 1, :c].float().cpu(), kr[:, h:h + 1, c:].float().cpu()
            vf[:, :, a0:a1], vf[:, :, b0:b1] = vr[:, h:h + 1, :c].float().cpu(), vr[:, h:h + 1, c:].float().cpu()
            del kr, vr
        sl = slice(4 * h, 4 * h + 4)
        r0, r1 = N - 256, N
        qf, gf = q[:, sl, rows - 256:].float().cpu(), do[:, sl, rows - 256:].float().cpu()
        s_ = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        s_.masked_fill_(torch.arange(N).view(1, -1) > torch.arange(r0, r1).view(-1, 1), float("-inf"))
        lse_ref = torch.logsumexp(s_, -1)
        p = torch.softmax(s_, -1)
        o_ref = torch.matmul(p, vf)
        ds = p * (torch.matmul(gf, vf.transpose(-1, -2)) - (gf * o_ref).sum(-1, keepdim=True))
        dq, dk, dv = keep["g"]
        res["sampled_error_vs_oracle"] = {
            "checked": "the last 256 rows of the sequence (rank 0's last rows), one KV-head group: O, LSE, dQ, and dK, dV of the last 256 keys",
            "o": orc.rel_max_err(keep["o"][:, sl, rows - 256:], o_ref),
            "lse_abs": orc.abs_max_err(keep["lse"][:, sl, rows - 256:], lse_ref),
            "dq": orc.rel_max_err(dq[:, sl, rows - 256:], torch.matmul(ds, kf) * scale),
            "dk": orc.rel_max_err(dk[:, h:h + 1, rows - 256:],
                                  (torch.matmul(ds[..., r0:r1].transpose(-1, -2), qf) * scale).sum(1, keepdim=True)),
            "dv": orc.rel_max_err(dv[:, h:h + 1, rows - 256:],
                                  torch.matmul(p[..., r0:r1].transpose(-1, -2), gf).sum(1, keepdim=True))}
    res["device_status"] = ext.device_status()
    return res


def run_sharded_legs(args, rank, world, local, dev, dist, ext, full_ms):
    peaks = measured_peaks()
    out = {}
    for name, fn in (("units_split", lambda: leg_units_split(args, rank, world, dev, dist, ext, full_ms)),
                     ("varlen_head_split", lambda: leg_varlen_split(args, rank, world, dev, dist, ext)),
                     ("decode_batch_split", lambda: leg_decode_split(args, rank, world, dev, dist, ext, peaks)),
                     ("long_context_ring", lambda: leg_ring(args, rank, world, local, dev, dist, ext))):
        try:
            out[name] = fn()
        except RuntimeError as e:
            # every rank must leave the leg: a failure on one rank is one on all (collectives inside)
            out[name] = {"error": str(e)[:300]}
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the CPU baseline and decode extras")
    ap.add_argument("--workload", default="gqa_fwd_bwd", choices=["gqa_fwd_bwd", "long_context", "varlen", "decode", "shape"],
                    help="secondary metrics.  long_context: B=1 Hq=32 Hkv=8 N=131072 d=128 causal forward+backward, "
                         "the sequence sharded over the ranks with the ring K/V exchange; varlen: 16 packed "
                         "sequences of 64..4096 tokens, H=16 d=128, heads dealt to the ranks; decode: batch 64 "
                         "split-K decode over a 32768-token cache, batch entries dealt to the ranks")
    ap.add_argument("--ring-layout", default="zigzag", choices=["zigzag", "contiguous"],
                    help="long_context with more than one rank: how the sequence rows are dealt to the ranks")
    ap.add_argument("--shape", action="append", default=[],
                    help="--workload shape: pass:B,Hq,Hkv,Nq,Nk,d[:noncausal] with pass = fwd | bwd | chunk | kvchunk; repeatable")
    ap.add_argument("--fwd-variant", type=int, default=0, choices=[0, 1, 2],
                    help="--workload shape: forward kernel variant (0 = the library's own choice, 1 = one query tile "
                         "per thread block, 2 = two tiles)")
    ap.add_argument("--decode-graph", action="store_true",
                    help="decode workload: replay one captured step as a CUDA graph instead of launching eagerly")
    ap.add_argument("--decode-batch", type=int, default=0,
                    help="decode workload on one rank: run this many of the 64 batch entries (what one of "
                         "64/N ranks holds), to see a shard's step without the other GPUs")
    ap.add_argument("--e2e-kv-heads-per-chunk", type=int, default=4, choices=[1, 2, 4, 8],
                    help="end-to-end leg: KV heads (with their query heads) of one batch entry per pipeline chunk")
    ap.add_argument("--kernel-source-hash", action="store_true",
                    help="print the hash an ncu capture record of the backward kernel must carry, and exit")
    ap.add_argument("--decode-profile", action="store_true",
                    help="run only a small decode case (batch 16, a few steps): the case profilers capture")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.kernel_source_hash:
        print(kernel_source_hash())
        return
    if args.impl == "reference":
        run_reference(args)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    rank, world, local, dist = dist_setup(args.gpus)
    import flash_attn_legacy_cuda as ext
    import flash_attn_legacy as fal

    if args.workload == "long_context":
        run_long_context(args, rank, world, local, dist, ext)
        return
    if args.workload == "varlen":
        run_varlen(args, rank, world, local, dist, ext)
        return
    if args.workload == "decode":
        run_decode(args, rank, world, local, dist, ext)
        return
    if args.workload == "shape":
        ext.set_forward_variant(args.fwd_variant)
        run_shapes(args, ext)
        return

    if args.decode_profile:
        res = run_decode_extra(ext, measured_peaks(), steps=max(args.steps, 4), batch=16)
        print(json.dumps({"decode_profile_case": res}))
        return

    w = WORKLOAD
    B, Hq, Hkv, N, d, causal = w["B"], w["Hq"], w["Hkv"], w["N"], w["d"], w["causal"]
    scale = 1.0 / math.sqrt(d)
    dev = torch.device("cuda", local)
    gen = torch.Generator(device="cuda").manual_seed(1 + rank)
    q = torch.randn(B, Hq, N, d, device=dev, generator=gen).half()
    k = torch.randn(B, Hkv, N, d, device=dev, generator=gen).half()
    v = torch.randn(B, Hkv, N, d, device=dev, generator=gen).half()
    do = torch.randn(B, Hq, N, d, device=dev, generator=gen).half()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, N, device=dev, dtype=torch.float32)
    grads = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    ws = torch.empty(ext.backward_workspace_bytes(B, Hq, N, d), dtype=torch.uint8, device=dev)
    fwd_flops, bwd_flops = step_flops()

    def step():
        ext.forward(q, k, v, scale, causal, out=o, lse=lse)
        ext.backward(do, q, k, v, o, lse, scale, causal, out=grads, workspace=ws)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident timing ----------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    ext.profile_enable(True)
    ext.profile_read(ext.KERNEL_FWD)
    ext.profile_read(ext.KERNEL_BWD)
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.mark_end()
    ms_total = e0.elapsed_time(e1)
    time.sleep(0.1)
    clocks = sampler.stop()
    fwd_ms, fwd_n = ext.profile_read(ext.KERNEL_FWD)
    bwd_ms, bwd_n = ext.profile_read(ext.KERNEL_BWD)
    ext.profile_enable(False)
    if dist is not None:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = t.item()
    ms_step = ms_total / args.steps
    value = world * (fwd_flops + bwd_flops) / (ms_step * 1e-3) / 1e12

    # ---------------- end to end from pinned host memory ------------------------
    hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
    h_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, k, v)]
    dq_, dk_, dv_ = q, k, v  # device staging buffers reused as H2D destinations

    # Eight chunks -- one batch entry x four KV heads (with their sixteen query heads) each --, three
    # streams: the copy-in of chunk c+1 and the copy-out of chunk c-1 run beside the kernels of chunk c
    # (the PCIe link is full duplex).  The copy-in stream sets the pace (336 MB per step); smaller chunks
    # shorten what cannot overlap -- the first chunk's copy-in, the last chunk's kernels and copy-out --
    # until the host's launch path becomes the limit (measured per step: 4 chunks 7.47 ms, 8 chunks
    # 6.70 ms, 16 chunks 7.42 ms, 32 chunks 14.5 ms).  Every chunk goes through the public autograd
    # operator on strided views: no staging copy.
    main_stream = torch.cuda.current_stream()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    kv_per_chunk = args.e2e_kv_heads_per_chunk
    group = Hq // Hkv
    chunks = [(b, kh, kh + kv_per_chunk) for b in range(B) for kh in range(0, Hkv, kv_per_chunk)]
    nchunk = len(chunks)
    computed = [None] * nchunk  # event: the kernels that read chunk c's staging buffers are done

    def e2e_step():
        for c, (b, k0, k1) in enumerate(chunks):
            bs, ks, qs = slice(b, b + 1), slice(k0, k1), slice(k0 * group, k1 * group)
            with torch.cuda.stream(s_in):
                if computed[c] is not None:
                    s_in.wait_event(computed[c])
                dq_[bs, qs].copy_(hq[bs, qs], non_blocking=True)
                dk_[bs, ks].copy_(hk[bs, ks], non_blocking=True)
                dv_[bs, ks].copy_(hv[bs, ks], non_blocking=True)
                do[bs, qs].copy_(hdo[bs, qs], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(loaded)
                qa = dq_[bs, qs].detach().requires_grad_(True)
                ka = dk_[bs, ks].detach().requires_grad_(True)
                va = dv_[bs, ks].detach().requires_grad_(True)
                out = fal.flash_attention(qa, ka, va, softmax_scale=scale, is_causal=causal)
                out.backward(do[bs, qs])
                computed[c] = torch.cuda.Event()
                computed[c].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[c])
                for dst, g, sl in zip(h_out, (qa.grad, ka.grad, va.grad), (qs, ks, ks)):
                    g.record_stream(s_out)
                    dst[bs, sl].copy_(g, non_blocking=True)

    def e2e_join():
        for st in (s_in, s_cmp, s_out):
            main_stream.wait_stream(st)

    for st in (s_in, s_cmp, s_out):
        st.wait_stream(main_stream)
    for _ in range(3):
        e2e_step()
    e2e_join()
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    e0.record()
    for st in (s_in, s_cmp, s_out):
        st.wait_stream(main_stream)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    e2e_ms /= e2e_steps
    e2e_value = world * (fwd_flops + bwd_flops) / (e2e_ms * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * t.element_size() for t in h_out)
    status = ext.device_status()

    # ---------------- roofline of the dominant kernel (backward main kernel) -----------
    peaks = measured_peaks()
    peak_tf = peaks["bf16_tflops"]
    roofline = None
    extra = {}
    traffic, traffic_source = recorded_traffic()
    if bwd_n:
        bwd_kernel_ms = bwd_ms / bwd_n
        achieved = bwd_flops / (bwd_kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "fal_bwd_kernel<128,causal>", "achieved": achieved,
                    "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
                    "traffic": traffic, "traffic_unit": "bytes per launch", "traffic_source": traffic_source,
                    "kernel_ms": bwd_kernel_ms, "frac_of_nominal_2250": achieved / 2250.0}
    if fwd_n:
        fwd_kernel_ms = fwd_ms / fwd_n
        fa = fwd_flops / (fwd_kernel_ms * 1e-3) / 1e12
        extra["fwd_kernel"] = {"kernel": "fal_fwd_kernel<128,causal>", "kernel_ms": fwd_kernel_ms,
                               "achieved_tflops": fa, "frac_of_measured_peak": fa / peak_tf,
                               "frac_of_nominal_2250": fa / 2250.0}

    # ---------------- the same step for several seconds (clocks settle under the power cap) ----------
    if world == 1 and not args.no_extras:
        sampler = ClockSampler(local)
        sampler.start()
        time.sleep(0.3)
        for _ in range(20):   # the reference's benchmark method: 20 warm-up iterations, then >= 100 timed
            step()
        torch.cuda.synchronize()
        n_sus = max(100, int(math.ceil(3000.0 / ms_step)))
        sampler.mark_begin()
        e0.record()
        for _ in range(n_sus):
            step()
        e1.record()
        torch.cuda.synchronize()
        sampler.mark_end()
        sus_ms = e0.elapsed_time(e1) / n_sus
        time.sleep(0.1)
        sus_clocks = sampler.stop()
        sus_tf = (fwd_flops + bwd_flops) / (sus_ms * 1e-3) / 1e12
        med, mx = sus_clocks.get("sm_mhz"), sus_clocks.get("sm_max_mhz")
        extra["sustained"] = {
            "steps": n_sus, "seconds": sus_ms * n_sus / 1e3, "ms_per_step": sus_ms, "tflops": sus_tf,
            "sm_mhz_median": med, "sm_max_mhz": mx, "reasons": sus_clocks.get("reasons"),
            "tflops_scaled_to_max_clock": sus_tf * mx / med if med and mx else None,
            "frac_of_sustained_peak": sus_tf / peaks["bf16_tflops_sustained"] if peaks.get("bf16_tflops_sustained") else None,
            "sustained_peak_tflops": peaks.get("bf16_tflops_sustained"),
            "peak_source": f"{peaks['source']} cuBLAS bf16, seconds-long loop"}
    if world > 1 and not args.no_extras:
        extra["sharded"] = run_sharded_legs(args, rank, world, local, dev, dist, ext, ms_step)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_extras:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
        tf, dt, threads, n_sl = cpu_baseline_sample(6, min_seconds=10.0)
        cpu_baseline = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"{n_sl} of 32 (batch, kv-head-group) slices of the same workload, {dt:.1f} s, "
                                  f"fp32 oracle forward + backward, os.cpu_count()={os.cpu_count()}"}
        try:
            extra["decode"] = run_decode_extra(ext, peaks)
        except RuntimeError as e:  # e.g. not enough free memory next to another job
            extra["decode"] = {"error": str(e)[:200]}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "global_batch": B * world, "per_gpu": w,
                       "l2_policy": "inputs+outputs per step (about 1 GB) exceed the 126 MB L2",
                       "parallelism": f"{world} x independent (batch, head-group) shards, no collective"},
            "per_gpu_tflops": value / world,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "pipeline": f"{nchunk} chunks of one batch entry x {kv_per_chunk} KV heads; copy-in, kernels and "
                                "copy-out on three streams"},
            "gpu_launches": 4 * args.steps,
            "launches_per_step": {"fal_fwd_kernel": 1, "fal_bwd_prep_kernel": 1, "fal_bwd_kernel": 1,
                                  "fal_bwd_post_kernel": 1},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "clocks": clocks,
            "device_status": status, "extra": extra,
        }))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
