"""Headline benchmark: training tokens/s of the 5B hybrid MoE on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events around exactly K
steps, barrier + synchronize on both sides, max over ranks) with the batch already on the
device; ``e2e`` repeats the measurement through the public step API with every step's
batch copied from pinned host memory and the step's loss read back to the host.
Synthetic data: uniform-random token ids from a seed; weights are random-init.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "train_tokens_per_sec_5b_hybrid_moe"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32, help="debug only: fewer layers (result flagged invalid)")
    ap.add_argument("--mamba-moe-mode", default="moe_ffn", choices=["moe_ffn", "routing_mamba"])
    ap.add_argument("--optimizer", default="muon", choices=["muon", "adamw"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ep-size", type=int, default=1,
                    help="expert-parallel group size (experts split over it; dense parameters stay data-parallel)")
    ap.add_argument("--moe-dtype", default="bf16", choices=["bf16", "mxfp8"], help="expert GEMM number format")
    ap.add_argument("--shard-params", action="store_true",
                    help="parameter-sharded plan (ZeRO-3 / FULL_SHARD, AdamW) instead of replicated parameters")
    ap.add_argument("--transport", default=None, choices=[None, "p2p", "nccl"],
                    help="gradient/parameter collectives: own NVLink peer kernels (default when available) or NCCL")
    return ap.parse_args()


MODEL_NAME = ("5B hybrid MoE (32L d2048 16/4 heads, 16 experts top-2 x16 MoE layers, "
              "Mamba d_state16, MoD 0.75, 4-token MTP, vocab 50304)")


def metric_name(args) -> str:
    """The headline metric for the bf16 replicated-parameter run; variants of the workload
    (MXFP8 experts, expert parallelism, parameter-sharded AdamW plan, reference Mamba+MoE
    semantics) are different benchmarks and carry their own metric names."""
    name = METRIC
    if args.mamba_moe_mode != "moe_ffn":
        name += "_routing_mamba"
    if args.moe_dtype != "bf16":
        name += f"_{args.moe_dtype}"
    if args.ep_size > 1:
        name += f"_ep{args.ep_size}"
    if args.shard_params:
        name += "_fullshard_adamw"
    return name


def workload_config(args, world: int, valid: bool) -> dict:
    """What is being measured, in the same words for both arms (arm-specific facts such as the
    parameter count, peak memory and transport go to ``detail``)."""
    return {"model": MODEL_NAME, "global_batch": args.micro_batch * world, "seq_len": args.seq_len,
            "parallelism": f"dp{world}", "mamba_moe_mode": args.mamba_moe_mode,
            "optimizer": "muon(2-D weights)+adamw" if args.optimizer == "muon" else "adamw",
            "l2": "inputs+weights (>11 GB) exceed L2 between iterations", "valid_config": valid}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_ours(args):
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    from kolmogorov_moe_architecture_b200.ops import cuda_ops

    world, rank, local = dist_setup(args)
    dev = torch.device("cuda", local)
    over = {}
    if args.layers != 32:
        L = args.layers
        over = dict(n_layers=L, moe_layers=tuple(i for i in range(L) if i % 4 in (1, 2)),
                    mamba_layers=tuple(i for i in range(L) if i % 4 == 1))
    mesh = None
    if args.ep_size > 1:
        from kolmogorov_moe_architecture_b200.parallel import mesh as pmesh
        mesh = pmesh.make_mesh(args.ep_size)
        over.update(moe_implementation="expert_parallel", ep_size=args.ep_size)
    if args.moe_dtype != "bf16":
        over.update(moe_dtype=args.moe_dtype)
    cfg = kmoe.get_bench_5b_config(mamba_moe_mode=args.mamba_moe_mode, max_seq_len=args.seq_len,
                                   use_gradient_checkpointing=False, **over)
    torch.manual_seed(0)
    with torch.device(dev):
        model = kmoe.MoETransformer(cfg, verbose=(rank == 0)).to(torch.bfloat16)
    n_params = sum(p.numel() for p in model.parameters())
    from kolmogorov_moe_architecture_b200.parallel.zero import ParallelPlan, ShardedDataParallel
    if args.shard_params:
        from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
        dp = FullyShardedDataParallel(model, lr=3e-4, transport=args.transport)
        transport = f"full-shard-{dp.transport}" + ("-overlap" if dp.overlap else "")
    else:
        dp = ShardedDataParallel(model, optimizer_kind=args.optimizer, transport=args.transport)
        transport = dp.transport
    if mesh is not None:
        experts = ShardedDataParallel(model, optimizer_kind="adamw", group=mesh.expert_dp_group, expert_params=True,
                                      grad_scale=1.0 / args.ep_size, broadcast_from_rank0=False, transport="nccl")
        dp = ParallelPlan([dp, experts])
    optimizer = dp.optimizer
    engine = TrainEngine(model, optimizer, grad_clip=1.0, dp=dp, device=dev)

    B, S = args.micro_batch, args.seq_len
    g = torch.Generator().manual_seed(1234 + rank)
    n_batches = 4
    host = [torch.randint(0, cfg.vocab_size, (B, S), generator=g).pin_memory() for _ in range(n_batches)]
    devb = [h.to(dev) for h in host]

    for i in range(args.warmup):
        engine.step(devb[i % n_batches])
    cuda_ops.check_status()
    barrier(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = cuda_ops.LAUNCHES["count"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        engine.step(devb[i % n_batches])
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    launches = cuda_ops.LAUNCHES["count"] - l0
    clocks = sampler.stop() if rank == 0 else {}
    cuda_ops.check_status()
    tokens = B * S * world * args.steps
    value = tokens / (ms / 1e3)

    e2e = None
    if not args.no_e2e:
        barrier(world)
        e0.record()
        last = 0.0
        for i in range(args.steps):
            st = engine.step(host[i % n_batches])        # H2D copy from pinned memory inside the step
            last = st.loss_value()                        # D2H read of the step's loss
        e1.record()
        barrier(world)
        ms2 = max_over_ranks(e0.elapsed_time(e1), world)
        e2e = {"value": tokens / (ms2 / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": B * S * 8,
               "d2h_bytes_per_step": 4, "ms_per_step": ms2 / args.steps, "last_loss": last}
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    if rank == 0:
        valid = args.layers == 32 and B == 4 and S == 2048
        if args.shard_params:
            args.optimizer = "adamw (sharded)"
        out = {
            "metric": metric_name(args), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours", "gpu_launches": launches, "clocks": clocks, "e2e": e2e,
            "config": workload_config(args, world, valid),
            "detail": {"params_b": round(n_params / 1e9, 3), "peak_mem_gb": round(peak_gb, 1),
                       "parallelism": (f"dp{world}" + (f"-{transport}" if args.shard_params else
                                                       (f"-zero1-{transport}" if world > 1 else ""))
                                       + (f"-ep{args.ep_size}-p2p" if args.ep_size > 1 else "")),
                       "optimizer": args.optimizer, "launches_per_step": launches / max(args.steps, 1)},
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        from baseline.run_reference import run_reference
        run_reference(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
