"""Small single-kernel workloads for Nsight Compute captures.

    python benchmarks/ncu_cases.py --case gemm|moe|attn|scan|adamw|ce|mxfp8 [--launches 4]

Each case holds well under 2 GB on the device, uses operands larger than L2 where the kernel is
bandwidth-sensitive, and launches the kernel of interest a handful of times so that
``ncu -k regex:<kernel> -s 2 -c 1`` captures a warm launch and the program then ends by itself.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--launches", type=int, default=4)
    a = ap.parse_args()
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c, eager
    bf = lambda *s, sc=0.05: (torch.randn(*s, device="cuda") * sc).to(torch.bfloat16)
    n = a.launches
    if a.case == "gemm":
        M, N, K = 8192, 8192, 2048
        x, w = bf(M, K), bf(N, K)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        for _ in range(n):
            c.mm_nt(x, w, out=out)
    elif a.case == "moe":
        T, d, f, E, k = 6144, 2048, 2816, 16, 2
        x = bf(T, d, sc=1.0).requires_grad_(True)
        w1, w2, w3 = bf(E, d, f).requires_grad_(True), bf(E, d, f).requires_grad_(True), bf(E, f, d).requires_grad_(True)
        wts, idx = eager.topk_softmax_route(torch.randn(T, E, device="cuda"), k)
        for _ in range(n):
            ops.grouped_swiglu(x, w1, w2, w3, idx, wts).backward(bf(T, d, sc=1.0))
    elif a.case == "attn":
        B, S, H, Hkv, D = 4, 2048, 16, 4, 128
        q, k_, v = bf(B, S, H, D, sc=1.0).requires_grad_(True), bf(B, S, Hkv, D, sc=1.0).requires_grad_(True), bf(B, S, Hkv, D, sc=1.0).requires_grad_(True)
        for _ in range(n):
            ops.attention(q, k_, v).backward(bf(B, S, H, D, sc=1.0))
    elif a.case == "scan":
        B, S, C, N = 4, 2048, 4096, 16
        u, dt, z = bf(B, S, C, sc=1.0).requires_grad_(True), bf(B, S, C, sc=1.0).requires_grad_(True), bf(B, S, C, sc=1.0).requires_grad_(True)
        A = (-torch.exp(torch.randn(C, N, device="cuda") * 0.5)).requires_grad_(True)
        Bm, Cm = bf(B, S, N, sc=1.0).requires_grad_(True), bf(B, S, N, sc=1.0).requires_grad_(True)
        D, bias = torch.randn(C, device="cuda", requires_grad=True), torch.randn(C, device="cuda", requires_grad=True)
        for _ in range(n):
            ops.selective_scan(u, dt, A, Bm, Cm, D, z, bias, True).backward(bf(B, S, C, sc=1.0))
    elif a.case == "adamw":
        N_ = 256 * 2**20
        p, g = bf(N_), bf(N_)
        m, v = torch.zeros(N_, device="cuda"), torch.zeros(N_, device="cuda")
        coef = torch.ones(1, device="cuda")
        for s in range(1, n + 1):
            torch.ops.kmoe.p2p_adamw_allgather([p.data_ptr()], g, m, v, 0, 1, 0, N_, 3e-4, 0.9, 0.95, 1e-8, 0.01, s, coef, 0)
    elif a.case == "ce":
        R, V = 2048, 50304
        logits = bf(R, V, sc=1.0)
        labels = torch.randint(0, V, (R,), device="cuda")
        gs = torch.full((1,), 1.0 / R, device="cuda")
        for _ in range(n):
            torch.ops.kmoe.ce_fwd_bwd(logits, labels, gs, -100, True)
    elif a.case == "mxfp8":
        from kolmogorov_moe_architecture_b200.ops import mxfp8 as mx
        M, N, K = 8192, 8192, 2048
        aq, sa = mx.quant_rows(bf(M, K, sc=1.0))
        bq, sb = mx.quant_rows(bf(N, K, sc=1.0))
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        for _ in range(n):
            mx.gemm_mx(aq, sa, bq, sb, out, M=M, N=N, K=K)
    else:
        raise SystemExit(f"unknown case {a.case}")
    torch.cuda.synchronize()
    c.check_status()
    print("ok", a.case)


if __name__ == "__main__":
    main()
