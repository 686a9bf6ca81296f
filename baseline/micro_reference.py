"""Microbenchmarks of the reference's own modules, for the per-kernel rows of the comparison table.

    python baseline/micro_reference.py [--which moe,attn,mod,mamba]

Runs the unmodified reference installed under ``baseline/_ref`` (nothing from this repository's
package is imported) on one GPU, at the shapes ``benchmarks/kernels.py`` uses for this library:

* ``moe``   - ``MoELayer`` forward+backward (``batched`` and, when importable, ``sparse``), 16384 tokens x 2048,
              16 experts of d_ff 4096, top-2 (moe_arch/model/moe.py:690-760).  The reference router sees random
              activations, so the expert loads are near uniform, and token-choice routing drops no token.
* ``attn``  - ``flash_attn_func`` with K/V expanded to the 16 query heads, as the reference's attention
              module calls it (moe_arch/model/attention.py:212-249): B=8, S=2048, 16 heads of 128.
* ``mod``   - ``MoDRouter`` forward+backward in eager PyTorch (moe_arch/model/mod.py:40-140), B=8, S=2048, d=2048.
* ``mamba`` - ``MambaBlock`` forward+backward (moe_arch/model/mamba.py:22-105; ``mamba_ssm`` when importable,
              else the reference's own SimpleSSM fallback), B=8, S=2048, d=2048.

Device-timed with CUDA events, three warm-up calls, a 256 MiB buffer written between timed calls (L2 flush),
median of 10.  One JSON line per row; a row that cannot run prints ``{"kernel": ..., "unavailable": why}``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
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
    return ts[len(ts) // 2]


def row(name, fn, flops=None, note=None):
    try:
        ms = timeit(fn)
        r = {"impl": "reference", "kernel": name, "ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
        if note:
            r["note"] = note
    except Exception as e:  # a missing kernel image or an out-of-memory error is a result, not a crash
        r = {"impl": "reference", "kernel": name, "unavailable": f"{type(e).__name__}: {e}".replace("\n", " ")[:200]}
    print(json.dumps(r), flush=True)


def config(**kw):
    from moe_arch.model.config import AdvancedMoEConfig
    base = dict(d_model=2048, n_layers=2, n_heads=16, n_kv_heads=4, head_dim=128, vocab_size=50304,
                max_seq_len=2048, n_experts=16, moe_top_k=2, d_ff_expert=4096, moe_layers=(0, 1),
                mamba_enabled=False, mamba_layers=(), mod_enabled=True)
    base.update(kw)
    return AdvancedMoEConfig(**base)


def bench_moe():
    from moe_arch.model.moe import MoELayer
    T, d, f, E, k = 16384, 2048, 4096, 16, 2
    fl = 3 * (2.0 * T * k * d * f * 3)
    for impl in ("batched", "sparse"):
        try:
            layer = MoELayer(config(moe_implementation=impl), 0).cuda().to(torch.bfloat16)
        except Exception as e:
            print(json.dumps({"impl": "reference", "kernel": f"MoELayer[{impl}]", "unavailable": str(e)[:200]}))
            continue
        x = torch.randn(8, T // 8, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        g = torch.randn_like(x)

        def fb():
            out = layer(x)
            out = out[0] if isinstance(out, tuple) else out
            out.backward(g)
            x.grad = None
            layer.zero_grad(set_to_none=True)
        row(f"MoELayer[{impl}] fwd+bwd, {T} tok x {d}, {E} experts d_ff {f}, top-{k}", fb, fl,
            note=type(layer.grouped_experts).__name__)
        del layer


def bench_attn():
    try:
        from flash_attn import flash_attn_func
    except Exception as e:
        print(json.dumps({"impl": "reference", "kernel": "flash_attn_func", "unavailable": str(e)[:200]}))
        return
    B, S, H, Hkv, D = 8, 2048, 16, 4, 128
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn_like(q)
    fl = 4.0 * B * H * S * S * D / 2

    def expand(t):      # the reference repeats K/V to the query heads before the call
        return t.unsqueeze(3).expand(B, S, Hkv, H // Hkv, D).reshape(B, S, H, D)

    def fwd():
        with torch.no_grad():
            flash_attn_func(q, expand(k), expand(v), causal=True)

    def fb():
        flash_attn_func(q, expand(k), expand(v), causal=True).backward(g)
        q.grad = k.grad = v.grad = None
    row(f"flash_attn_func (K/V expanded to {H} heads) fwd B={B}", fwd, fl)
    row(f"flash_attn_func (K/V expanded to {H} heads) fwd+bwd B={B}", fb, 3.5 * fl)


def bench_mod():
    from moe_arch.model.mod import MoDRouter
    B, S, d = 8, 2048, 2048
    r = MoDRouter(config()).cuda().to(torch.bfloat16)
    x = torch.randn(B, S, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)

    def fb():
        out = r(x)
        (out[1].float().sum() + out[2].float().sum()).backward()
        x.grad = None
        r.zero_grad(set_to_none=True)
    row(f"MoDRouter (eager) fwd+bwd B={B} S={S} d={d}", fb)


def bench_mamba():
    from moe_arch.model.mamba import MambaBlock
    B, S, d = 8, 2048, 2048
    blk = MambaBlock(config(mamba_enabled=True, mamba_layers=(0,), moe_layers=(1,))).cuda().to(torch.bfloat16)
    inner = type(getattr(blk, "mamba", blk)).__name__
    x = torch.randn(B, S, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn_like(x)

    def fb():
        blk(x).backward(g)
        x.grad = None
        blk.zero_grad(set_to_none=True)
    row(f"MambaBlock fwd+bwd B={B} S={S} d={d}", fb, note=f"mixer: {inner}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", default="moe,attn,mod,mamba")
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "moe_arch")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    sys.path.insert(0, REF)
    table = {"moe": bench_moe, "attn": bench_attn, "mod": bench_mod, "mamba": bench_mamba}
    for w in a.which.split(","):
        try:
            table[w]()
        except Exception as e:
            print(json.dumps({"impl": "reference", "kernel": w, "unavailable": f"{type(e).__name__}: {e}"[:300]}),
                  flush=True)


if __name__ == "__main__":
    main()
