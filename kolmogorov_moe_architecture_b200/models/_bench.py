"""Timing helper of the module-level benchmarks (``benchmark_*`` functions of the MoE variants)."""
from __future__ import annotations

import time
from typing import Callable, Dict

import torch


def default_device() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def time_ms(fn: Callable[[], object], device: str, warmup: int = 5, iters: int = 20) -> float:
    """Milliseconds per call: CUDA events after warm-up with a synchronize on both sides on a GPU, host clock
    on the CPU."""
    for _ in range(warmup):
        fn()
    if str(device).startswith("cuda"):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / max(iters, 1)
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) / max(iters, 1) * 1e3


def routed_inputs(n_tokens: int, d_model: int, n_experts: int, top_k: int, device: str, dtype, seed: int = 0):
    """(x, expert indices (T, k) distinct per token, weights (T, k) summing to one)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_tokens, d_model, generator=g).to(device=device, dtype=dtype)
    w, idx = torch.topk(torch.softmax(torch.randn(n_tokens, n_experts, generator=g), -1), top_k, dim=-1)
    return x, idx.to(device), (w / w.sum(-1, keepdim=True)).to(device=device, dtype=dtype)


def report(title: str, times: Dict[str, float], base: str) -> Dict[str, float]:
    print(title)
    for name, t in times.items():
        print(f"  {name:28s} {t:9.3f} ms   {times[base] / t:6.2f}x")
    return times
