"""Multi-GPU training (counterpart of the reference's ``train_distributed.py``).

    torchrun --nproc_per_node=8 train_distributed.py --config configs/training_4.5b.yaml

One process per GPU over NCCL.  By default parameters are replicated in bf16; reduced gradients and
optimizer state are sharded by whole tensors (one reduce-scatter and one all-gather per step,
run by this library's NVLink peer kernels when peer access is available, NCCL otherwise).
``--shard-params`` selects the reference's regime instead (parameters sharded per block, gathered
around each block's forward and backward, AdamW on the shards, optional ``--cpu-offload``).
``moe_implementation: expert_parallel`` in the YAML shards the experts over an expert-parallel
group with differentiable dispatch/combine.  Adds what the reference's script lacks: seeding,
global-norm clipping across shards, Muon, sharded checkpoints and ``--resume``.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# helpers that the reference's launcher defines at module level and other code imports from it
from kolmogorov_moe_architecture_b200.training.script_api import (  # noqa: E402,F401
    PackedSequenceDataset, check_parameter_gradients, cleanup_distributed, collect_router_stats, create_dataloader,
    create_model, create_optimizer, create_scheduler, load_config, load_tokenizer, print_debug_stats,
    setup_distributed, train_step, wrap_model_with_fsdp)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Distributed MoE Training")
    ap.add_argument("--config", type=str, required=True)
    ap.add_argument("--resume", type=str, default=None)
    ap.add_argument("--shard-params", action="store_true",
                    help="shard the parameters per block over the ranks (ZeRO-3 / FULL_SHARD, AdamW) instead of "
                         "replicating them; for models that do not fit one GPU")
    ap.add_argument("--cpu-offload", action="store_true",
                    help="with --shard-params: keep the shards and optimizer state in pinned host memory")
    ap.add_argument("--no-activation-checkpointing", action="store_true")
    ap.add_argument("--activation-checkpointing", action="store_true",
                    help="recompute blocks in backward (off by default: 180 GB of HBM holds the activations)")
    ap.add_argument("--8bit-optimizer", action="store_true", dest="use_8bit_optimizer")
    ap.add_argument("--debug", action="store_true")
    ap.add_argument("--debug-interval", type=int, default=100)
    ap.add_argument("--use-ddp", action="store_true", help="accepted for compatibility; same replicated-parameter plan")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--transport", default=None, choices=[None, "p2p", "nccl"])
    ap.add_argument("--checkpoint-dir", type=str, default=None)
    ap.add_argument("--jsonl", type=str, default=None)
    ap.add_argument("--async-checkpoint", action="store_true",
                    help="copy checkpoint state to pinned host memory and write the files in the background")
    a = ap.parse_args(argv)
    from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
    spec = RunSpec(config_path=a.config, steps=a.steps, resume=a.resume, weights="bf16", checkpoint_format="C",
                   checkpoint_dir=a.checkpoint_dir, grad_checkpoint=a.activation_checkpointing,
                   data_mode="synthetic" if a.synthetic else "streaming", debug=a.debug, debug_interval=a.debug_interval,
                   transport=a.transport, jsonl=a.jsonl, shard_params=a.shard_params or a.cpu_offload,
                   cpu_offload=a.cpu_offload, async_checkpoint=a.async_checkpoint,
                   use_8bit_optimizer=a.use_8bit_optimizer)
    return run_training(spec)


if __name__ == "__main__":
    main()
