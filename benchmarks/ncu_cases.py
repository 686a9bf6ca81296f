"""Small single-kernel workloads for Nsight Compute captures.

    python benchmarks/ncu_cases.py --case gemm|moe|attn|scan|adamw|allgather|ce|mxfp8|mod|ep_dispatch|ep_gemm2 [--launches 4]

Each case holds well under 2 GB on the device, uses operands larger than L2 where the kernel is
bandwidth-sensitive, and launches the kernel of interest a handful of times so that
``ncu --clock-control none -k regex:<kernel> -s 2 -c 1 ...`` captures a warm launch and the program then
ends by itself (one process, one GPU; without ``--clock-control none`` ncu would lock the GPU clocks).
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
    ap.add_argument("--shape", default=None, help="gemm case: M,N,K (default 8192,8192,2048)")
    a = ap.parse_args()
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c, eager
    bf = lambda *s, sc=0.05: (torch.randn(*s, device="cuda") * sc).to(torch.bfloat16)
    n = a.launches
    if a.case == "gemm":
        M, N, K = (int(v) for v in a.shape.split(",")) if a.shape else (8192, 8192, 2048)
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
    elif a.case == "allgather":
        # the parameter-gather kernel of the sharded plan in a one-rank "group": it reads a shard and stores it
        # into the gather buffer (with more ranks the same stores go to every peer's buffer)
        N_ = 256 * 2**20
        shard, buf = bf(N_), torch.empty(N_, dtype=torch.bfloat16, device="cuda")
        for blocks in (32, 0)[: max(1, min(2, n))]:
            for _ in range(max(1, n // 2)):
                torch.ops.kmoe.p2p_allgather([buf.data_ptr()], 0, 1, 0, N_, 0, shard, blocks)
    elif a.case == "ce":
        R, V = 2048, 50304
        logits = bf(R, V, sc=1.0)
        labels = torch.randint(0, V, (R,), device="cuda")
        gs = torch.full((1,), 1.0 / R, device="cuda")
        for _ in range(n):
            torch.ops.kmoe.ce_fwd_bwd(logits, labels, gs, -100, True)
    elif a.case in ("ep_dispatch", "ep_gemm2"):
        # the expert-parallel kernels in a one-rank group (the "peer" pointers are this GPU's own buffers), so a
        # single process can be profiled: dispatch (permute + exchange) and GEMM 2 with the row-pointer epilogue
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29711")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        from kolmogorov_moe_architecture_b200.parallel import ep_p2p
        K = torch.ops.kmoe
        T, d, f, E, k = 16384, 2048, 4096, 16, 2
        x = bf(T, d, sc=1.0)
        wts, idx = eager.topk_softmax_route(torch.randn(T, E, device="cuda"), k)
        buf = ep_p2p.get_buffers(T, k, d, E, torch.bfloat16, x.device, None)
        pos, row_src, counts, offsets, _tg, _m = K.moe_plan(idx.reshape(-1).contiguous(), None, E, 0)
        for _ in range(n):
            K.ep_dispatch(x, row_src, None, offsets, counts, buf.recv_ptrs, buf.meta_ptrs, 0, 1, E, buf.cap, k)
        buf.barrier()
        meta_in = buf.meta.clone()
        R = buf.max_rows_exp
        slot_dst, offs_l, tile_group, meta_l = K.ep_recv_plan(meta_in, E, 1, R)
        Xp = torch.empty(R, d, dtype=torch.bfloat16, device="cuda")
        row_ptr = torch.empty(R, dtype=torch.int64, device="cuda")
        K.ep_move(buf.recv, Xp, meta_in, slot_dst, offs_l, buf.ret_ptrs, 0, E, 1, buf.cap, 0, row_ptr)
        H, w3 = bf(R, f, sc=1.0), bf(E, f, d)
        for _ in range(n):
            c.gemm(H, w3, Xp, mode=c.GROUPED_M, M=R, N=d, Kd=f, groups=E, b_major=c.MAJ_MN, lda=f, ldb=d, ldc=d,
                   b_gs=f * d, tile_group=tile_group, num_m_tiles=meta_l[0:1], row_ptr=row_ptr)
        torch.cuda.synchronize()
        c.check_status()
        ep_p2p.release_buffers()
        dist.destroy_process_group()
    elif a.case == "mod":
        B, S, k, d = 4, 2048, 1536, 2048
        h, res = bf(B, S, d, sc=1.0).requires_grad_(True), bf(B, S, d, sc=1.0).requires_grad_(True)
        idx = torch.stack([torch.randperm(S, device="cuda")[:k].sort().values for _ in range(B)])
        w = torch.rand(B, k, device="cuda").to(torch.bfloat16).requires_grad_(True)
        for _ in range(n):
            ops.mod_combine(res, ops.mod_gather(h, idx), w, idx).backward(bf(B, S, d, sc=1.0))
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
