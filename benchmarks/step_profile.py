"""Per-kernel breakdown of one training step of the benchmark model (torch.profiler device times).

    python benchmarks/step_profile.py [--layers 32] [--steps 2] [--top 60] [--mamba-moe-mode moe_ffn]

Builds the 5B hybrid model of ``bench.py`` (or fewer layers of it), runs three warm-up steps through the
public ``TrainEngine`` / ``ShardedDataParallel`` path and profiles ``--steps`` steps.  Prints the sum of device
time per kernel name and step, the number of launches, and - separately - the optimizer ranges.  Kernels on the
side stream (the AdamW update overlaps Newton-Schulz) are counted at their own duration, so the sum exceeds the
step time; ranges such as ``Optimizer.step#Muon.step`` are annotations, listed apart and not part of the sum.
One process, one GPU.
"""
import argparse
import collections
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--top", type=int, default=60)
    ap.add_argument("--mamba-moe-mode", default="moe_ffn")
    a = ap.parse_args()
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    from torch.profiler import ProfilerActivity, profile

    L = a.layers
    cfg = kmoe.get_bench_5b_config(n_layers=L, moe_layers=tuple(i for i in range(L) if i % 4 in (1, 2)),
                                   mamba_layers=tuple(i for i in range(L) if i % 4 == 1),
                                   use_gradient_checkpointing=False, mamba_moe_mode=a.mamba_moe_mode)
    dev = torch.device("cuda", 0)
    with torch.device(dev):
        model = kmoe.MoETransformer(cfg, verbose=False).to(torch.bfloat16)
    dp = ShardedDataParallel(model)
    eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, dp=dp, device=dev)
    ids = torch.randint(0, cfg.vocab_size, (4, 2048), device=dev)
    for _ in range(3):
        eng.step(ids)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.step(ids)
    e1.record()
    torch.cuda.synchronize()
    print(f"step time without the profiler: {e0.elapsed_time(e1) / a.steps:.1f} ms")
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(a.steps):
            eng.step(ids)
        torch.cuda.synchronize()
    kern = collections.defaultdict(lambda: [0.0, 0])
    ranges = collections.defaultdict(lambda: [0.0, 0])
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        t = e.device_time_total if hasattr(e, "device_time_total") else e.cuda_time_total
        tgt = ranges if ("#" in e.name or e.name.startswith("Optimizer")) else kern
        tgt[e.name][0] += t
        tgt[e.name][1] += 1
    n = a.steps
    tot = sum(v[0] for v in kern.values())
    print(f"sum of kernel time per step: {tot / n / 1e3:.2f} ms; kernels per step: {sum(v[1] for v in kern.values()) / n:.0f}")
    for name, (t, c) in sorted(kern.items(), key=lambda kv: -kv[1][0])[: a.top]:
        print(f"{t / n / 1e3:9.3f} ms {100 * t / tot:5.1f}% {c / n:7.0f}x  {name[:140]}")
    for name, (t, c) in sorted(ranges.items(), key=lambda kv: -kv[1][0]):
        print(f"range {t / n / 1e3:9.3f} ms {c / n:5.0f}x  {name[:120]}")


if __name__ == "__main__":
    main()
