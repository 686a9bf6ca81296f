"""Per-kernel microbenchmarks with roofline fractions.

    python benchmarks/kernels.py [--which gemm,moe,attn,scan,ce,norm] [--out file.jsonl]

Timing: CUDA events, 3 warm-up + 10 timed launches, L2 flushed between launches by writing
a 256 MB buffer.  Fractions are of the measured peaks in MEASURED_PEAKS.json (fallback
6.65 TB/s, 1.59 PFLOP/s).  Counterpart of the reference's kernel benchmark harness
(moe_arch/kernels/benchmark.py:96-169), which times only the expert FFN.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_flush = None


def timeit(fn, iters=10, warm=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 2**20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def report(rows, name, secs, flops=None, bytes_=None, extra=None):
    bw, fl, kind = peaks()
    r = {"kernel": name, "ms": round(secs * 1e3, 4)}
    if flops:
        r["tflops"] = round(flops / secs / 1e12, 1)
        r[f"frac_of_{kind}_bf16_peak"] = round(flops / secs / fl, 3)
    if bytes_:
        r["gbs"] = round(bytes_ / secs / 1e9, 1)
        r[f"frac_of_{kind}_hbm"] = round(bytes_ / secs / bw, 3)
    if extra:
        r.update(extra)
    rows.append(r)
    print(json.dumps(r), flush=True)


def bench_gemm(rows):
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c
    bf = lambda *s: (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)
    for (M, N, K) in [(8192, 2048, 2048), (8192, 8192, 2048), (8192, 5632, 2048), (8192, 2048, 5632),
                      (8192, 50304, 2048), (4096, 4096, 4096)]:
        a, b = bf(M, K), bf(N, K)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        fl = 2.0 * M * N * K
        report(rows, f"kmoe.mm_nt {M}x{N}x{K}", timeit(lambda: c.mm_nt(a, b, out=out)), fl)
        report(rows, f"cublas.mm_nt {M}x{N}x{K}", timeit(lambda: torch.matmul(a, b.t(), out=out)), fl)
    M, N, K = 8192, 2048, 50304
    a, b = bf(M, K), bf(K, N)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    report(rows, f"kmoe.mm_nn {M}x{N}x{K}", timeit(lambda: c.mm_nn(a, b, out=out)), 2.0 * M * N * K)
    report(rows, f"cublas.mm_nn {M}x{N}x{K}", timeit(lambda: torch.matmul(a, b, out=out)), 2.0 * M * N * K)
    M, N, K = 50304, 2048, 8192
    a, b = bf(K, M), bf(K, N)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    report(rows, f"kmoe.mm_tn {M}x{N}x{K}", timeit(lambda: c.mm_tn(a, b, out=out)), 2.0 * M * N * K)
    report(rows, f"cublas.mm_tn {M}x{N}x{K}", timeit(lambda: torch.matmul(a.t(), b, out=out)), 2.0 * M * N * K)
    c.check_status()


def bench_moe(rows):
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c, eager
    for (T, d, f, E, k, tag) in [(6144, 2048, 2816, 16, 2, "5B layer"), (16384, 2048, 4096, 16, 2, "microbench")]:
        x = (torch.randn(T, d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
        w1 = (torch.randn(E, d, f, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
        w2 = (torch.randn(E, d, f, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
        w3 = (torch.randn(E, f, d, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
        bias = torch.log(1.0 / torch.arange(1, E + 1, device="cuda").float())       # Zipf(1) loads
        logits = torch.randn(T, E, device="cuda") + bias
        wts, idx = eager.topk_softmax_route(logits, k)
        go = torch.randn(T, d, device="cuda").to(torch.bfloat16)
        fl_f = 2.0 * T * k * 3 * d * f

        def fwd():
            return ops.grouped_swiglu(x, w1, w2, w3, idx, wts)

        def fwdbwd():
            out = fwd()
            out.backward(go)
            x.grad = w1.grad = w2.grad = w3.grad = None
        report(rows, f"moe_ffn fwd ({tag}) T={T} E={E} top{k} zipf", timeit(fwd), fl_f)
        report(rows, f"moe_ffn fwd+bwd ({tag})", timeit(fwdbwd), 3 * fl_f)
    c.check_status()


def bench_mxfp8(rows):
    """Block-scaled fp8 GEMM alone (operands already quantised), the quantisers, and the expert FFN on it.
    Fractions are against the bf16 cuBLAS peak, so 1.0 means "as fast as a perfect bf16 GEMM"."""
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c, eager, mxfp8 as mx
    for (M, N, K) in [(8192, 8192, 2048), (12288, 2816, 2048), (8192, 8192, 8192)]:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        aq, sa = mx.quant_rows(a)
        bq, sb = mx.quant_rows(b)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        report(rows, f"gemm mxfp8 {M}x{N}x{K}", timeit(lambda: mx.gemm_mx(aq, sa, bq, sb, out, M=M, N=N, K=K)),
               2.0 * M * N * K)
        report(rows, f"quant_rows {M}x{K}", timeit(lambda: mx.quant_rows(a)), None, M * K * 3.0)
        report(rows, f"quant_cols {M}x{K}", timeit(lambda: mx.quant_cols(a)), None, M * K * 3.0)
    T, d, f, E, k = 6144, 2048, 2816, 16, 2
    x = (torch.randn(T, d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    w1 = (torch.randn(E, d, f, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
    w2 = (torch.randn(E, d, f, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
    w3 = (torch.randn(E, f, d, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
    logits = torch.randn(T, E, device="cuda") + torch.log(1.0 / torch.arange(1, E + 1, device="cuda").float())
    wts, idx = eager.topk_softmax_route(logits, k)
    go = torch.randn(T, d, device="cuda").to(torch.bfloat16)
    fl_f = 2.0 * T * k * 3 * d * f
    for dt in ("mxfp8", "bf16"):
        def fwd():
            return ops.grouped_swiglu(x, w1, w2, w3, idx, wts, None, dt)

        def fwdbwd():
            fwd().backward(go)
            x.grad = w1.grad = w2.grad = w3.grad = None
        report(rows, f"moe_ffn {dt} fwd (5B layer)", timeit(fwd), fl_f)
        report(rows, f"moe_ffn {dt} fwd+bwd (5B layer)", timeit(fwdbwd), 3 * fl_f)
    c.check_status()


def bench_attn(rows):
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c
    import torch.nn.functional as F
    for B in (4, 8):
        S, H, Hkv, D = 2048, 16, 4, 128
        q = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
        k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
        v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
        go = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16)
        fl = 4.0 * B * H * S * S * D / 2

        def fb():
            o = ops.attention(q, k, v)
            o.backward(go)
            q.grad = k.grad = v.grad = None

        def lib():
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=True, enable_gqa=True)
            o.backward(go.transpose(1, 2))
            q.grad = k.grad = v.grad = None
        report(rows, f"kmoe.attention fwd B={B}", timeit(lambda: ops.attention(q, k, v)), fl)
        report(rows, f"kmoe.attention fwd+bwd B={B}", timeit(fb), 3.5 * fl)
        report(rows, f"sdpa(cudnn) fwd+bwd B={B}", timeit(lib), 3.5 * fl)
    c.check_status()


def bench_attn_docs(rows):
    """Packed documents (mean length 512) on the flash kernels against the same call without boundaries."""
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import eager
    B, S, H, Hkv, D = 4, 2048, 16, 4, 128
    q = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    go = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16)
    doc_ids = torch.arange(S, device="cuda").div(512, rounding_mode="floor").expand(B, S).contiguous()
    ds = eager.doc_start_from_ids(doc_ids)

    def run(doc):
        o = ops.attention(q, k, v, doc_start=doc)
        o.backward(go)
        q.grad = k.grad = v.grad = None
    fl = 3.5 * 4.0 * B * H * S * S * D / 2
    report(rows, "kmoe.attention fwd+bwd B=4, 4 packed documents of 512", timeit(lambda: run(ds)), fl / 4)
    report(rows, "kmoe.attention fwd+bwd B=4, one document", timeit(lambda: run(None)), fl)


def bench_scan(rows):
    from kolmogorov_moe_architecture_b200 import ops
    for B in (4, 8):
        S, C, N = 2048, 4096, 16
        u = torch.randn(B, S, C, device="cuda").to(torch.bfloat16).requires_grad_(True)
        dt = torch.randn(B, S, C, device="cuda").to(torch.bfloat16).requires_grad_(True)
        z = torch.randn(B, S, C, device="cuda").to(torch.bfloat16).requires_grad_(True)
        A = (-torch.exp(torch.randn(C, N, device="cuda") * 0.5)).requires_grad_(True)
        Bm = torch.randn(B, S, N, device="cuda").to(torch.bfloat16).requires_grad_(True)
        Cm = torch.randn(B, S, N, device="cuda").to(torch.bfloat16).requires_grad_(True)
        D = torch.randn(C, device="cuda", requires_grad=True)
        bias = torch.randn(C, device="cuda", requires_grad=True)
        go = torch.randn(B, S, C, device="cuda").to(torch.bfloat16)
        byt = 4.0 * B * S * C * 2

        def f():
            return ops.selective_scan(u, dt, A, Bm, Cm, D, z, bias, True)

        def fb():
            f().backward(go)
        with torch.no_grad():
            report(rows, f"selective_scan fwd B={B}", timeit(f), None, byt)
        report(rows, f"selective_scan fwd+bwd B={B}", timeit(fb), None, byt * 2.75)
        xz = torch.randn(B, S, 2 * C, device="cuda").to(torch.bfloat16).requires_grad_(True)
        w = torch.randn(C, 4, device="cuda", requires_grad=True)
        b = torch.randn(C, device="cuda", requires_grad=True)

        def cf():
            ops.causal_conv1d(xz[..., :C], w, b, True).backward(go)
        report(rows, f"causal_conv1d fwd+bwd B={B}", timeit(cf), None, 5.0 * B * S * C * 2)


def bench_ce(rows):
    from kolmogorov_moe_architecture_b200 import ops
    B, S, d, V = 4, 2048, 2048, 50304
    h = (torch.randn(B, S, d, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    Ws = [(torch.randn(V, d, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True) for _ in range(4)]
    labels = torch.randint(0, V, (B, S), device="cuda")

    def fb():
        tot, _ = ops.mtp_cross_entropy(h, Ws, labels, (0.5, 0.25, 0.15, 0.1))
        tot.backward()
        h.grad = None
        for w in Ws:
            w.grad = None
    report(rows, "lm_head+mtp_ce fwd+bwd (4 heads, 8192 tok)", timeit(fb, iters=5), 4 * 3 * 2.0 * B * S * d * V)


def bench_muon(rows):
    """Newton-Schulz orthogonalisation (5 cubic iterations) on the stacked matrix shapes of the 5B model:
    per iteration a symmetric Gram product (upper-triangle tiles only) and a product with the
    ``1.5 Y - 0.5 G Y`` epilogue.  FLOPs counted as executed: 5 * (g^2 o + 2 g^2 o), g = min(m, n), o = max."""
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c
    for (b, m, n, tag) in [(48, 5632, 2048, "dense FFN w1/w2"), (16, 2048, 5632, "dense FFN w3 (16 of 48)"),
                           (48, 2048, 2048, "attention q/o"), (48, 512, 2048, "attention k/v"),
                           (8, 8192, 2048, "mamba in_proj"), (8, 2048, 4096, "mamba out_proj")]:
        x = torch.randn(b, m, n, device="cuda").to(torch.bfloat16)
        sumsq = x.float().pow(2).sum(dim=(1, 2))
        g_, o_ = min(m, n), max(m, n)
        fl = b * 5 * 3.0 * g_ * g_ * o_
        report(rows, f"newton_schulz x5 ({tag}) {b}x{m}x{n}", timeit(lambda: ops.newton_schulz(x, 5, sumsq)), fl)
    c.check_status()


def bench_norm(rows):
    from kolmogorov_moe_architecture_b200 import ops
    x = torch.randn(8192, 2048, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = torch.ones(2048, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn_like(x)
    byt = 8192 * 2048 * 2
    with torch.no_grad():
        report(rows, "rmsnorm fwd 8192x2048", timeit(lambda: ops.rmsnorm(x, w, 1e-5)), None, 2 * byt)
    report(rows, "rmsnorm fwd+bwd 8192x2048", timeit(lambda: ops.rmsnorm(x, w, 1e-5).backward(go)), None, 5 * byt)


def bench_modules(rows):
    """Whole modules at the shapes of the reference-side table (``baseline/micro_reference.py``): the MoE layer
    with its router, the MoD router and the Mamba block, forward + backward."""
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    from kolmogorov_moe_architecture_b200.models.moe import MoELayer
    from kolmogorov_moe_architecture_b200.models.mod import MoDRouter
    from kolmogorov_moe_architecture_b200.models.mamba import MambaBlock
    cfg = AdvancedMoEConfig(d_model=2048, n_layers=2, n_heads=16, n_kv_heads=4, head_dim=128, vocab_size=50304,
                            max_seq_len=2048, n_experts=16, moe_top_k=2, d_ff_expert=4096, moe_layers=(1,),
                            mamba_enabled=True, mamba_layers=(0,), mod_enabled=True)
    T, d, f, k = 16384, 2048, 4096, 2
    x = torch.randn(8, T // 8, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    g = torch.randn_like(x)

    def fb(mod, pick=lambda o: o):
        def run():
            o = mod(x)
            pick(o).backward(g) if pick(o).shape == g.shape else pick(o).backward()
            x.grad = None
            mod.zero_grad(set_to_none=True)
        return run
    moe = MoELayer(cfg, 1).cuda().to(torch.bfloat16)
    report(rows, f"MoELayer fwd+bwd, {T} tok x {d}, 16 experts d_ff {f}, top-{k}",
           timeit(fb(moe, lambda o: o[0] if isinstance(o, tuple) else o)), 3 * (2.0 * T * k * d * f * 3))
    del moe
    mod = MoDRouter(cfg).cuda().to(torch.bfloat16)
    report(rows, "MoDRouter fwd+bwd B=8 S=2048 d=2048",
           timeit(fb(mod, lambda o: o[1].float().sum() + o[2].float().sum())))
    mamba = MambaBlock(cfg).cuda().to(torch.bfloat16)
    report(rows, "MambaBlock fwd+bwd B=8 S=2048 d=2048", timeit(fb(mamba)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", default="gemm,moe,mxfp8,attn,scan,ce,norm,muon")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    rows = []
    table = {"gemm": bench_gemm, "moe": bench_moe, "mxfp8": bench_mxfp8, "attn": bench_attn, "attn_docs": bench_attn_docs, "scan": bench_scan, "ce": bench_ce,
             "norm": bench_norm, "muon": bench_muon, "modules": bench_modules}
    for k in a.which.split(","):
        table[k](rows)
    if a.out:
        with open(a.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
