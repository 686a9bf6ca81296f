"""Expert-choice combine benchmark (counterpart of the reference's ``tools/benchmark_expert_choice.py``): the
weighted scatter-add of (B, E, C, d) expert outputs back to (B, S, d)

* as a Python loop over (batch, expert) with ``index_add_``            (the reference's original form),
* as one vectorised ``scatter_add``                                     (the reference's default),
* through this framework's deterministic combine kernel on a GPU: the slots are turned into the token-choice
  bookkeeping with k = E (``pos[t, e]`` = row of token t at expert e, or -1) and every token sums its own rows,
  no atomics (what ``GroupedExpertsExpertChoice`` runs; the reference's third form is a Triton atomic-add kernel),
* optionally (``--with-compile``) the vectorised form under ``torch.compile``,

checks that they agree to 1e-4 (1e-2 for the bf16 kernel) and prints the time per call.

    python tools/benchmark_expert_choice.py [--device cuda] [--batch-size 4] [--seq-len 2048] [--d-model 1024]
        [--n-experts 16] [--capacity-factor 1.25] [--warmup 10] [--iters 100]
"""
import argparse
import math
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def scatter_loop(output, weighted_outputs, token_indices):
    out, w_out, idx = output, weighted_outputs, token_indices
    B, E, C, d = w_out.shape
    for b in range(B):
        for e in range(E):
            out[b].index_add_(0, idx[b, e], w_out[b, e])
    return out


def scatter_vectorised(output, weighted_outputs, token_indices):
    out, w_out, idx = output, weighted_outputs, token_indices
    B, E, C, d = w_out.shape
    return out.scatter_add(1, idx.reshape(B, E * C, 1).expand(-1, -1, d), w_out.reshape(B, E * C, d))


def make_kernel_combine(w_out, idx, S):
    """The framework's kernel path for the same sum: rows ordered (expert, batch, slot) in bf16, the position table
    of every (token, expert) pair, and a closure that runs the combine kernel.  Needs distinct tokens per
    (batch, expert), which is what expert-choice routing produces."""
    K = torch.ops.kmoe
    B, E, C, d = w_out.shape
    dev = w_out.device
    T = B * S
    t_glob = idx + (torch.arange(B, device=dev) * S).view(B, 1, 1)
    a_rows = (t_glob * E + torch.arange(E, device=dev).view(1, E, 1)).permute(1, 0, 2).reshape(-1)
    pos = torch.full((T * E,), -1, dtype=torch.int32, device=dev)
    pos[a_rows] = torch.arange(E * B * C, dtype=torch.int32, device=dev)
    ones = torch.zeros(T * E, dtype=torch.float32, device=dev)
    ones[a_rows] = 1.0
    Y = w_out.permute(1, 0, 2, 3).reshape(E * B * C, d).to(torch.bfloat16).contiguous()

    def run(out, _w, _i):
        return K.moe_combine(Y, pos, ones, T, E).view(B, S, d)
    return run


def time_fn(fn, out_like, w_out, idx, warmup: int, iters: int) -> float:
    sync = torch.cuda.synchronize if out_like.is_cuda else (lambda: None)
    for _ in range(warmup):
        fn(torch.zeros_like(out_like), w_out, idx)
    sync()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn(torch.zeros_like(out_like), w_out, idx)
    sync()
    return (time.perf_counter() - t0) / max(iters, 1) * 1e3


# the reference's names for the two PyTorch forms and the timer
original_scatter_add = scatter_loop
vectorized_scatter_add = scatter_vectorised


def benchmark_fn(fn, output, weighted_outputs, token_indices, warmup: int = 10, iters: int = 100) -> float:
    """Milliseconds per call of ``fn(zeros_like(output), weighted_outputs, token_indices)``."""
    return time_fn(fn, output, weighted_outputs, token_indices, warmup, iters)


def main(argv=None):
    ap = argparse.ArgumentParser(description="expert-choice combine: loop, scatter_add, kernel")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cuda", "cpu"])
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--n-experts", type=int, default=16)
    ap.add_argument("--capacity-factor", type=float, default=1.25)
    ap.add_argument("--with-compile", action="store_true", help="also time the vectorised form under torch.compile")
    a = ap.parse_args(argv)
    dev = a.device
    if dev == "cuda" and not torch.cuda.is_available():
        print("CUDA not available, using the CPU")
        dev = "cpu"
    B, S, E, d = a.batch_size, a.seq_len, a.n_experts, a.d_model
    C = min(S, int(math.ceil(S * a.capacity_factor / E)))
    print(f"device {dev}  batch {B}  seq {S}  d_model {d}  experts {E}  capacity {C}  pairs per sequence {E * C}")
    g = torch.Generator().manual_seed(0)
    w_out = torch.randn(B, E, C, d, generator=g).to(dev)
    # every expert picks C distinct tokens of each sequence, as the router's top-k over tokens does
    idx = torch.stack([torch.stack([torch.randperm(S, generator=g)[:C] for _ in range(E)]) for _ in range(B)]).to(dev)
    zero = torch.zeros(B, S, d, device=dev)
    variants = [("loop", scatter_loop), ("scatter_add", scatter_vectorised)]
    if dev == "cuda" and d % 8 == 0:
        try:
            from kolmogorov_moe_architecture_b200.ops import ext_available
            if ext_available():
                variants.append(("kernel (bf16)", make_kernel_combine(w_out, idx, S)))
        except Exception as e:
            print(f"kernel variant unavailable: {type(e).__name__}: {e}")
    if a.with_compile:
        try:
            variants.append(("compiled", torch.compile(scatter_vectorised)))
        except Exception as e:
            print(f"torch.compile unavailable: {type(e).__name__}: {e}")
    ref = scatter_loop(torch.zeros_like(zero), w_out, idx)
    times = {}
    for name, fn in variants:
        try:
            got = fn(torch.zeros_like(zero), w_out, idx).float()
            tol = 1e-2 * float(ref.abs().max()) if "bf16" in name else 1e-4
            ok = torch.allclose(got, ref, atol=tol, rtol=1e-4 if "bf16" not in name else 1e-2)
            times[name] = time_fn(fn, zero, w_out, idx, a.warmup, a.iters)
            print(f"{name:14s} {times[name]:9.4f} ms   {times['loop'] / times[name]:6.2f}x   "
                  f"{'PASS' if ok else 'FAIL (max diff %.3g)' % float((got - ref).abs().max())}")
            assert ok, f"{name} disagrees with the loop"
        except AssertionError:
            raise
        except Exception as e:
            print(f"{name:14s} failed: {type(e).__name__}: {e}")
    return times


if __name__ == "__main__":
    main()
