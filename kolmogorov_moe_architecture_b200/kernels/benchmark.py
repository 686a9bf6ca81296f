"""Grouped-SwiGLU kernel against its plain PyTorch definition: agreement and time, on the four shapes of the
reference's harness (reference: moe_arch/kernels/benchmark.py:163-169 - (experts, d_model, d_ff, tokens) =
(8, 512, 1024, 1024), (16, 768, 2048, 2048), (48, 1024, 3096, 4096), (64, 1536, 4096, 8192), top-2).

    python -m kolmogorov_moe_architecture_b200.kernels.benchmark [--device cuda] [--iters 20] [--with-backward]

Times are device times (CUDA events, after warm-up, synchronised on both sides) on a GPU and host times on the
CPU, where only the PyTorch definition runs.  The reference's third shape has d_ff = 3096, which is not a multiple
of 64; this library's GEMM wants that, so the shape is run at d_ff = 3136 and the substitution is printed.
"""
from __future__ import annotations

import argparse
import time
from typing import Dict, Tuple

import torch

from . import grouped_swiglu_forward, grouped_swiglu_forward_pytorch, grouped_swiglu_with_grad, is_kernel_available

SHAPES = [(8, 512, 1024, 1024, 2), (16, 768, 2048, 2048, 2), (48, 1024, 3096, 4096, 2), (64, 1536, 4096, 8192, 2)]


def create_test_data(n_experts: int, d_model: int, d_ff: int, n_tokens: int, top_k: int = 2, device=None,
                     dtype=None, seed: int = 0) -> Tuple[torch.Tensor, ...]:
    """(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends): ``n_tokens * top_k`` rows sorted by the
    expert they go to (stable), the stacked expert weights, and each expert's row range."""
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if str(device).startswith("cuda") else torch.float32)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_tokens, d_model, generator=g)
    experts = torch.randint(0, n_experts, (n_tokens * top_k,), generator=g)
    tokens = torch.arange(n_tokens).repeat_interleave(top_k)
    order = torch.argsort(experts, stable=True)
    ends = torch.cumsum(torch.bincount(experts, minlength=n_experts), 0)
    starts = ends - torch.bincount(experts, minlength=n_experts)
    w = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(device=device, dtype=dtype)
    return (x[tokens[order]].to(device=device, dtype=dtype), w(n_experts, d_model, d_ff), w(n_experts, d_model, d_ff),
            w(n_experts, d_ff, d_model), experts[order].to(device), starts.to(device), ends.to(device))


def verify_correctness(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends, tol: float = 0.1) -> bool:
    """Kernel against the PyTorch definition (fp32 on the same bf16 inputs): max |difference| below ``tol``."""
    ref = grouped_swiglu_forward_pytorch(sorted_inputs.float(), W1.float(), W2.float(), W3.float(),
                                         sorted_expert_ids, seg_starts, seg_ends)
    if not (sorted_inputs.is_cuda and is_kernel_available()):
        print("  kernel not available on this device: nothing to compare")
        return True
    got = grouped_swiglu_forward(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends).float()
    diff = (got - ref).abs()
    ok = float(diff.max()) < tol
    print(f"  max |diff| {float(diff.max()):.5f}  mean |diff| {float(diff.mean()):.6f}  {'ok' if ok else 'MISMATCH'}")
    return ok


def _time(fn, n_warmup: int, n_iters: int, cuda: bool) -> float:
    for _ in range(n_warmup):
        fn()
    if cuda:
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n_iters
    t0 = time.perf_counter()
    for _ in range(n_iters):
        fn()
    return (time.perf_counter() - t0) / n_iters * 1e3


def benchmark(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends, n_warmup: int = 5,
              n_iters: int = 20, with_backward: bool = False) -> Dict[str, float]:
    """Milliseconds per call of the PyTorch loop and, on a GPU with the library loaded, of the kernel path
    (forward, and forward + backward through ``grouped_swiglu_with_grad`` when asked)."""
    cuda = sorted_inputs.is_cuda
    args = (sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends)
    out = {"pytorch_ms": _time(lambda: grouped_swiglu_forward_pytorch(*args), n_warmup, n_iters, cuda)}
    print(f"  PyTorch loop   {out['pytorch_ms']:9.3f} ms")
    if cuda and is_kernel_available():
        out["kernel_ms"] = _time(lambda: grouped_swiglu_forward(*args), n_warmup, n_iters, True)
        rows, d, f = sorted_inputs.shape[0], W1.shape[1], W1.shape[2]
        tflops = 6.0 * rows * d * f / (out["kernel_ms"] * 1e-3) / 1e12
        print(f"  kernel         {out['kernel_ms']:9.3f} ms   {out['pytorch_ms'] / out['kernel_ms']:6.2f}x   "
              f"{tflops:7.1f} TFLOP/s")
        if with_backward:
            xs = sorted_inputs.detach().requires_grad_(True)
            ws = [w.detach().requires_grad_(True) for w in (W1, W2, W3)]

            def step():
                grouped_swiglu_with_grad(xs, *ws, sorted_expert_ids).sum().backward()
            out["kernel_fwd_bwd_ms"] = _time(step, n_warmup, n_iters, True)
            print(f"  kernel fwd+bwd {out['kernel_fwd_bwd_ms']:9.3f} ms")
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="grouped SwiGLU: kernel against the PyTorch definition")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--with-backward", action="store_true")
    ap.add_argument("--shapes", default=None, help="'E,d,f,T,k;...' instead of the four standard shapes")
    a = ap.parse_args(argv)
    shapes = ([tuple(int(v) for v in s.split(",")) for s in a.shapes.split(";")] if a.shapes else SHAPES)
    print(f"device {a.device}; kernel available: {is_kernel_available()}")
    results = []
    for E, d, f, T, k in shapes:
        f_run = f if f % 64 == 0 or not str(a.device).startswith("cuda") else (f + 63) // 64 * 64
        note = f" (d_ff {f} run as {f_run}: multiples of 64)" if f_run != f else ""
        print(f"{E} experts, d_model {d}, d_ff {f_run}, {T} tokens, top-{k}: {T * k} rows{note}")
        data = create_test_data(E, d, f_run, T, k, device=a.device)
        ok = verify_correctness(*data)
        results.append({"shape": (E, d, f_run, T, k), "ok": ok,
                        **benchmark(*data, n_warmup=a.warmup, n_iters=a.iters, with_backward=a.with_backward)})
    return results


if __name__ == "__main__":
    main()
