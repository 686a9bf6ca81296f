"""Expert-parallel MoE layer microbenchmark (forward + backward), one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/ep_layer.py [--tokens 16384 --d-model 2048 --d-ff 4096 --experts 16 --top-k 2]

Every rank holds ``tokens`` tokens and E / N experts; routing is Zipf(1.0)-skewed over the experts.
Reports, timed with CUDA events on the device and reduced with max over ranks:
  * the layer on the peer-pointer transport (dispatch kernel, grouped GEMMs, GEMM 2 storing into the
    source ranks) and on the all_to_all transport (NCCL),
  * the dispatch kernel alone and GEMM 2 with / without the peer-pointer epilogue, with the bytes that
    cross NVLink, so each fused path can be set against its roofline
    max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s per direction).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0          # measured peer copy bandwidth per direction per GPU on this pool
BF16_TFLOPS = 1647.5        # measured cuBLAS bf16 burst


def timed(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--capacity-factor", type=float, default=1.25,
                    help="each source rank keeps at most cf * tokens * k / E assignments per expert (0 = no dropping)")
    ap.add_argument("--moe-dtype", default="bf16", choices=["bf16", "mxfp8"],
                    help="number format of the expert GEMMs (rows cross NVLink in bf16 either way)")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as C
    from kolmogorov_moe_architecture_b200.parallel import ep, ep_p2p

    T, d, f, E, k = a.tokens, a.d_model, a.d_ff, a.experts, a.top_k
    nl = E // ws
    torch.manual_seed(7 + rank)
    bf = lambda *s, sc=0.02: (torch.randn(*s, device="cuda") * sc).to(torch.bfloat16)
    x = bf(T, d, sc=1.0).requires_grad_(True)
    w1, w2, w3 = bf(nl, d, f).requires_grad_(True), bf(nl, d, f).requires_grad_(True), bf(nl, f, d).requires_grad_(True)
    logits = torch.randn(T, E, device="cuda") + torch.log(1.0 / torch.arange(1, E + 1, device="cuda").float())
    wts, idx = torch.softmax(logits, -1).topk(k, dim=-1)
    wts = wts.to(torch.bfloat16).requires_grad_(True)
    go = bf(T, d, sc=1.0)
    keep = None
    if a.capacity_factor > 0:
        import math
        keep = ops.capacity_keep_mask(idx, E, int(math.ceil(a.capacity_factor * T * k / E)))

    def clear():
        x.grad = w1.grad = w2.grad = w3.grad = wts.grad = None

    def fused():
        ep_p2p.expert_parallel_ffn_fused(x, idx, wts, w1, w2, w3, E, None, keep, moe_dtype=a.moe_dtype).backward(go)
        clear()

    def fused_fwd():
        with torch.no_grad():
            ep_p2p.expert_parallel_ffn_fused(x, idx, wts, w1, w2, w3, E, None, keep, moe_dtype=a.moe_dtype)

    local_fn = lambda xx, ii, ww, kk: ops.grouped_swiglu(xx, w1, w2, w3, ii, ww, kk, a.moe_dtype)

    def a2a():
        ep.expert_parallel_ffn(x, idx, wts, local_fn, E, None, keep=keep).backward(go)
        clear()

    def a2a_fwd():
        with torch.no_grad():
            ep.expert_parallel_ffn(x, idx, wts, local_fn, E, None, keep=keep)

    kept = idx.numel() if keep is None else int(keep.sum().item())
    kept_t = torch.tensor([float(kept)], device="cuda")
    dist.all_reduce(kept_t)
    flops_fwd = 2.0 * (kept_t.item() / ws) * 3 * d * f   # mean per rank; the busiest rank does more (see live rows)
    res = {"world": ws, "tokens_per_rank": T, "d_model": d, "d_ff": f, "experts": E, "top_k": k,
           "capacity_factor": a.capacity_factor, "moe_dtype": a.moe_dtype, "kept_assignments_mean_per_rank": kept_t.item() / ws}
    for name, fn, mult in (("fused_p2p fwd", fused_fwd, 1), ("fused_p2p fwd+bwd", fused, 3),
                           ("all_to_all fwd", a2a_fwd, 1), ("all_to_all fwd+bwd", a2a, 3)):
        ms = timed(fn)
        res[name + " ms"] = round(ms, 4)
        res[name + " TFLOP/s per GPU"] = round(mult * flops_fwd / ms / 1e9, 1)
    C.check_status()

    # the two fused kernels by themselves
    K = torch.ops.kmoe
    buf = ep_p2p.get_buffers(T, k, d, E, torch.bfloat16, x.device, None)
    pos, row_src, counts, offsets, _tg, _m = K.moe_plan(idx.reshape(-1).contiguous(),
                                                        keep.reshape(-1) if keep is not None else None, E, 0)
    xc = x.detach().contiguous()

    def dispatch_only():
        K.ep_dispatch(xc, row_src, None, offsets, counts, buf.recv_ptrs, buf.meta_ptrs, buf.rank, ws, E, buf.cap, k)
    ms = timed(dispatch_only)
    buf.barrier()
    meta_in = buf.meta.clone()
    # bytes over NVLink: rows this rank sends to other ranks (egress) and receives from them (ingress);
    # the kernel cannot finish before the busiest port of any rank has moved its bytes
    cnt = counts.view(ws, nl).sum(1).float()
    egress = (cnt.sum() - cnt[rank]) * d * 2
    slot_cnt = meta_in.view(nl, ws, 2)[:, :, 0].sum(0).float()
    ingress = (slot_cnt.sum() - slot_cnt[rank]) * d * 2
    port = torch.stack([egress, ingress]).max().reshape(1)
    dist.all_reduce(port, op=dist.ReduceOp.MAX)
    t_roof_d = port.item() / (NVLINK_GBS * 1e6)
    res["dispatch kernel ms"] = round(ms, 4)
    res["dispatch busiest NVLink port MB"] = round(port.item() / 1e6, 1)
    res["dispatch roofline ms"] = round(t_roof_d, 4)
    res["dispatch frac of roofline"] = round(t_roof_d / ms, 3)

    R = buf.max_rows_exp
    slot_dst, offs_l, tile_group, meta_l = K.ep_recv_plan(meta_in, nl, ws, R)
    Xp = torch.empty(R, d, dtype=torch.bfloat16, device="cuda")
    row_ptr = torch.empty(R, dtype=torch.int64, device="cuda")
    K.ep_move(buf.recv, Xp, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 0, row_ptr)
    H = bf(R, f, sc=1.0)
    Y = torch.empty(R, d, dtype=torch.bfloat16, device="cuda")
    live = int(meta_l[1].item())
    kw = dict(mode=C.GROUPED_M, M=R, N=d, Kd=f, groups=nl, b_major=C.MAJ_MN, lda=f, ldb=d, ldc=d, b_gs=f * d,
              tile_group=tile_group, num_m_tiles=meta_l[0:1])
    w3d = w3.detach()
    ms_local = timed(lambda: C.gemm(H, w3d, Y, **kw))
    ms_peer = timed(lambda: C.gemm(H, w3d, Y, row_ptr=row_ptr, **kw))
    fl = 2.0 * live * d * f
    t_loc = torch.tensor([max(fl / (BF16_TFLOPS * 1e9), ingress.item() / (NVLINK_GBS * 1e6)),
                          egress.item() / (NVLINK_GBS * 1e6)], device="cuda")   # results go back the way rows came
    dist.all_reduce(t_loc, op=dist.ReduceOp.MAX)
    t_roof = t_loc.max().item()                                             # ms
    res["gemm2 local store ms"] = round(ms_local, 4)
    res["gemm2 + combine transfer (peer epilogue) ms"] = round(ms_peer, 4)
    res["gemm2+combine roofline ms"] = round(t_roof, 4)
    res["gemm2+combine frac of roofline"] = round(t_roof / ms_peer, 3)
    res["live rows on rank 0"] = live
    C.check_status()
    if rank == 0:
        print(json.dumps(res, indent=1), flush=True)
        if a.out:
            with open(a.out, "w") as fh:
                json.dump(res, fh, indent=1)
    dist.barrier()
    ep_p2p.release_buffers()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
