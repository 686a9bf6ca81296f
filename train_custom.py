"""Custom loop with packed documents (counterpart of the reference's ``train_custom.py``).

    python train_custom.py --config configs/training_4.5b.yaml [--profile] [--no-packing]
    torchrun --nproc_per_node=8 train_custom.py --config ...

Streams documents, packs them into fixed-length rows with per-token document ids, masks
labels that would cross a document boundary, optionally restricts attention to the own
document (``data.use_document_attention_mask``), prefetches batches into pinned memory from a
background thread, and writes format-C checkpoint directories (newest three kept).
``--profile`` reports a data / step time breakdown measured with CUDA events.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# helpers that the reference's script defines at module level and other code imports from it
from kolmogorov_moe_architecture_b200.data.dolma_dataset import ThreadedPrefetcher  # noqa: E402,F401
from kolmogorov_moe_architecture_b200.training.script_api import (  # noqa: E402,F401
    CosineWarmupScheduler, CUDAPrefetcher, PackedSequenceDataset, StandardDataset, TimingStats, TrainConfig,
    cleanup_distributed, compute_loss, compute_token_weights, create_dataloader, evaluate, is_main_process,
    load_checkpoint, print_rank0, save_checkpoint, setup_distributed, setup_fsdp)


def train(config):
    """Train from a ``TrainConfig`` (reference: train_custom.py:944-1295): the configuration's YAML file drives the
    run, its fields override the file's step count, batch size, checkpoint directory and loss weighting."""
    from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
    assert config.config_path, "TrainConfig.from_yaml(path) records the file the run is built from"
    spec = RunSpec(config_path=config.config_path, steps=config.max_steps, batch_size=config.batch_size,
                   strict_config=True, weights="bf16" if config.dtype == "bfloat16" else "fp32_autocast",
                   optimizer_family="muon8bit_all" if config.optimizer == "muon" else "adamw", checkpoint_format="C",
                   checkpoint_dir=config.checkpoint_dir,
                   data_mode="packed" if config.pack_sequences else "streaming",
                   document_mask=bool(config.use_document_attention_mask), wandb=bool(config.use_wandb),
                   profile=bool(config.profile), compile=bool(config.compile),
                   token_weight_decay=config.token_weight_decay if config.use_token_weights or config.token_weight_decay
                   else 0.0)
    return run_training(spec)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Custom MoE Training Script")
    ap.add_argument("--config", type=str, required=True)
    ap.add_argument("--resume", type=str, default=None)
    ap.add_argument("--wandb", action="store_true")
    ap.add_argument("--no-packing", action="store_true")
    ap.add_argument("--compile", action="store_true")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--batch-size", type=int, default=None)
    ap.add_argument("--gpu", type=int, default=None)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--checkpoint-dir", type=str, default=None)
    ap.add_argument("--jsonl", type=str, default=None, help="also write metrics to this JSONL file")
    ap.add_argument("--token-weight-decay", type=float, default=0.0,
                    help="> 0: weigh later positions more in the loss (also: training.use_token_weights / "
                         "training.token_weight_decay in the config)")
    a = ap.parse_args(argv)
    from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, section
    data = section(load_yaml(a.config), "data")
    spec = RunSpec(config_path=a.config, steps=a.steps, batch_size=a.batch_size, resume=a.resume, strict_config=True,
                   weights="bf16", optimizer_family="muon8bit_all" if section(load_yaml(a.config), "optimizer").get(
                       "type") == "muon" else "adamw", checkpoint_format="C", checkpoint_dir=a.checkpoint_dir,
                   data_mode="synthetic" if a.synthetic else ("streaming" if a.no_packing else "packed"),
                   document_mask=bool(data.get("use_document_attention_mask")), wandb=a.wandb, gpu=a.gpu,
                   profile=a.profile, compile=a.compile, jsonl=a.jsonl,
                   token_weight_decay=a.token_weight_decay)
    return run_training(spec)


if __name__ == "__main__":
    main()
