"""Single-GPU training (counterpart of the reference's ``train.py``).

    python train.py --config configs/production_training.yaml --steps 50000 --batch-size 4 --seq-len 2048

Regime: bf16 (or fp16) weights, Muon-on-matrices + AdamW or grouped AdamW per the YAML
``optimizer.type``, constant learning rate, format-B checkpoints under
``<checkpoint-dir>/<config name>/checkpoint-{N}[-interrupted|-final].pt``, SIGINT/SIGTERM saves an
``-interrupted`` checkpoint, periodic router-collapse probe, ``--reallocate`` to re-seed collapsed
routers from healthy layers, ``--resume`` to continue from a checkpoint.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# helpers that the reference's script defines at module level and other code imports from it
from kolmogorov_moe_architecture_b200.training.script_api import (  # noqa: E402,F401
    check_router_collapse_fast, get_cache_path, get_dataloader, get_model_state_dict, load_config, signal_handler)
from kolmogorov_moe_architecture_b200.training.script_api import save_state_checkpoint as save_checkpoint  # noqa: E402,F401
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, default="configs/production_training.yaml")
    ap.add_argument("--steps", type=int, default=50000)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--compile", action="store_true", help="accepted for compatibility; the kernels are already fused")
    ap.add_argument("--wandb", action="store_true")
    ap.add_argument("--wandb-project", type=str, default="Kolmogorov-Testing")
    ap.add_argument("--wandb-run", type=str, default=None)
    ap.add_argument("--grad-accum", type=int, default=8)
    ap.add_argument("--grad-checkpoint", action="store_true")
    ap.add_argument("--max-examples", type=int, default=200000)
    ap.add_argument("--checkpoint-dir", type=str, default="./checkpoints")
    ap.add_argument("--save-interval", type=int, default=5000)
    ap.add_argument("--resume", type=str, default=None)
    ap.add_argument("--precision", type=str, default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--no-pack", action="store_true")
    ap.add_argument("--low-memory", action="store_true")
    ap.add_argument("--lr-scale", type=float, default=1.0)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--reallocate", action="store_true")
    ap.add_argument("--entropy-threshold", type=float, default=0.85)
    ap.add_argument("--balanced-routing", action="store_true")
    ap.add_argument("--collapse-check-interval", type=int, default=50)
    ap.add_argument("--collapse-entropy-threshold", type=float, default=0.7)
    ap.add_argument("--synthetic", action="store_true", help="train on uniform-random token ids")
    ap.add_argument("--jsonl", type=str, default=None, help="also write metrics to this JSONL file")
    a = ap.parse_args(argv)
    from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
    spec = RunSpec(config_path=a.config, steps=a.steps, batch_size=a.batch_size, seq_len=a.seq_len,
                   grad_accum=a.grad_accum, weights=a.precision, optimizer_family="auto", checkpoint_format="B",
                   checkpoint_dir=a.checkpoint_dir, save_interval=a.save_interval, resume=a.resume,
                   data_mode="synthetic" if a.synthetic else ("streaming" if a.no_pack else "auto"),
                   grad_checkpoint=a.grad_checkpoint, compile=a.compile, wandb=a.wandb, wandb_project=a.wandb_project,
                   wandb_run=a.wandb_run, lr_scale=a.lr_scale, gpu=a.gpu, balanced_routing=a.balanced_routing,
                   collapse_check_interval=a.collapse_check_interval,
                   collapse_entropy_threshold=a.collapse_entropy_threshold, reallocate=a.reallocate,
                   entropy_threshold=a.entropy_threshold, constant_lr=True, jsonl=a.jsonl)
    return run_training(spec)


if __name__ == "__main__":
    main()
