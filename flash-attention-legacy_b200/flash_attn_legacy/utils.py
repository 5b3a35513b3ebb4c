"""Device information and a small A/B timing helper.

Same public names as flash_attn_legacy/utils.py of the reference
(`get_device_info`, `check_gpu_compatibility`, `benchmark_flash_vs_standard`),
re-targeted: the only supported device is compute capability 10.x (B200).
"""
from typing import Dict, Optional

import torch

_ARCH_NAMES = {
    60: "Pascal", 61: "Pascal", 70: "Volta", 75: "Turing", 80: "Ampere", 86: "Ampere",
    89: "Ada Lovelace", 90: "Hopper", 100: "Blackwell (B200)", 103: "Blackwell (B300)",
    120: "Blackwell (consumer)",
}


def get_device_info(device: Optional[int] = None) -> Dict:
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA not available")
    if device is None:
        device = torch.cuda.current_device()
    props = torch.cuda.get_device_properties(device)
    sm = props.major * 10 + props.minor
    supported = props.major == 10
    return {
        "name": props.name,
        "sm_version": sm,
        "arch": _ARCH_NAMES.get(sm, f"Unknown (SM {sm})"),
        "total_memory_gb": round(props.total_memory / (1024 ** 3), 2),
        "shared_mem_per_block": getattr(props, "shared_memory_per_block_optin",
                                        getattr(props, "shared_memory_per_block", 0)),
        "multiprocessor_count": props.multi_processor_count,
        "has_tensor_cores": sm >= 70,
        "kernel_path": ("sm_100a path: tcgen05 tensor cores, TMEM accumulators, TMA"
                        if supported else "Unsupported (compute capability 10.x required)"),
        "supported": supported,
    }


def check_gpu_compatibility(device: Optional[int] = None, verbose: bool = True) -> bool:
    if not torch.cuda.is_available():
        if verbose:
            print("CUDA is not available")
        return False
    info = get_device_info(device)
    if verbose:
        print(f"GPU: {info['name']}")
        print(f"Architecture: {info['arch']} (SM {info['sm_version']})")
        print(f"Memory: {info['total_memory_gb']} GB")
        print(f"SMs: {info['multiprocessor_count']}")
        print(f"Shared Mem/Block: {info['shared_mem_per_block']} bytes")
        print(f"Kernel path: {info['kernel_path']}")
        verdict = "[OK] supported" if info["supported"] else "[FAIL] needs compute capability 10.x"
        print(f"\n{verdict}: {info['name']}")
    return info["supported"]


def _time_ms(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters, torch.cuda.max_memory_allocated() / 1e6


def benchmark_flash_vs_standard(batch_size: int = 2, num_heads: int = 8, seq_len: int = 2048,
                                head_dim: int = 64, is_causal: bool = False,
                                num_warmup: int = 10, num_iters: int = 100) -> Dict:
    """Times flash_attention against materialised fp32-softmax attention on the same inputs."""
    from .flash_attn import flash_attention

    dev = torch.device("cuda")
    q = torch.randn(batch_size, num_heads, seq_len, head_dim, device=dev, dtype=torch.float16)
    k, v = torch.randn_like(q), torch.randn_like(q)
    scale = head_dim ** -0.5

    def eager():
        s = torch.matmul(q.float(), k.float().transpose(-2, -1)) * scale
        if is_causal:
            s.masked_fill_(torch.triu(torch.ones(seq_len, seq_len, device=dev, dtype=torch.bool), 1),
                           float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1).half(), v)

    flash_ms, flash_mem = _time_ms(lambda: flash_attention(q, k, v, is_causal=is_causal),
                                   num_warmup, num_iters)
    std_ms, std_mem = _time_ms(eager, num_warmup, num_iters)
    return {
        "config": f"B={batch_size} H={num_heads} N={seq_len} d={head_dim}",
        "flash_ms": round(flash_ms, 3), "std_ms": round(std_ms, 3),
        "speedup": round(std_ms / flash_ms, 2) if flash_ms > 0 else 0,
        "flash_mem_mb": round(flash_mem, 1), "std_mem_mb": round(std_mem, 1),
        "mem_savings_pct": round((1 - flash_mem / std_mem) * 100, 1) if std_mem > 0 else 0,
    }
