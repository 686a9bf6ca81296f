"""Library-trainer entrypoint (counterpart of the reference's ``scripts/train.py``): fp32 master
weights with bf16 autocast, hybrid Muon/AdamW or AdamW, cosine schedule with warm-up, the
``Trainer`` loop with format-A checkpoints; Ctrl-C saves ``checkpoint_interrupted.pt``.

    python scripts/train.py --config configs/test.yaml [--max_steps N] [--device cpu]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from kolmogorov_moe_architecture_b200.training.script_api import load_config  # noqa: E402,F401


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, required=True)
    ap.add_argument("--resume", type=str, default=None)
    ap.add_argument("--max_steps", type=int, default=None)
    ap.add_argument("--device", type=str, default=None)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--wandb", action="store_true")
    a = ap.parse_args(argv)
    import torch
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.data import TokenizerWrapper, get_dataloaders
    from kolmogorov_moe_architecture_b200.training.lr_schedule import get_lr_scheduler
    from kolmogorov_moe_architecture_b200.training.muon_optimizer import get_muon_optimizer
    from kolmogorov_moe_architecture_b200.training.optim_factory import make_adamw
    from kolmogorov_moe_architecture_b200.training.trainer import Trainer
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_strict, section
    y = load_yaml(a.config)
    tc, oc, dc = section(y, "training"), section(y, "optimizer"), section(y, "data")
    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    cfg = model_config_strict(y)
    model = MoETransformer(cfg).to(device)
    if oc.get("type") == "muon":
        opt = get_muon_optimizer(model, lr=tc["max_lr"], momentum=oc.get("momentum", 0.95),
                                 weight_decay=oc.get("weight_decay", 0.01), fsdp_mode=False)
    else:
        opt = make_adamw(model.parameters(), tc["max_lr"], weight_decay=oc.get("weight_decay", 0.01))
    sched = get_lr_scheduler(opt, tc["total_tokens"], tc["batch_size"], cfg.max_seq_len, tc["warmup_steps"],
                             tc["max_lr"], tc["min_lr_ratio"])
    tok = None if a.synthetic else TokenizerWrapper(dc.get("tokenizer_name", "gpt2"), vocab_size=cfg.vocab_size)
    tr, va = get_dataloaders(tok, cfg, batch_size=tc["batch_size"], num_workers=dc.get("num_workers", 0),
                             use_memory_mapped=dc.get("use_memory_mapped", False), data_path=dc.get("data_path"),
                             synthetic=a.synthetic)
    trainer = Trainer(model, opt, sched, tr, va, y, device=device, use_amp=device == "cuda",
                      gradient_accumulation_steps=tc["gradient_accumulation_steps"],
                      gradient_clip_norm=tc["gradient_clip_norm"], checkpoint_dir=tc["checkpoint_dir"],
                      log_interval=tc["log_interval"], eval_interval=tc["eval_interval"],
                      save_interval=tc["save_interval"], use_wandb=a.wandb)
    if a.resume:
        trainer.load_checkpoint(a.resume)
    try:
        trainer.train(max_steps=a.max_steps)
    except KeyboardInterrupt:
        trainer.save_checkpoint("checkpoint_interrupted.pt")
    return trainer


if __name__ == "__main__":
    main()
