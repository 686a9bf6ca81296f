"""HuggingFace-Trainer entrypoint (counterpart of the reference's ``train_production.py``).

    python train_production.py --config configs/training_500m_hf.yaml [--max_steps N] [--synthetic]

The model is wrapped by ``MoEModelWrapper``; HF owns the loop, logging and ``checkpoint-N/``
directories (``save_total_limit=3``); the optimizer is the hybrid Muon/AdamW or AdamW and the
schedule the cosine-with-warm-up of this library.  ``mixed_precision.fp8: true`` selects the
block-scaled fp8 expert GEMMs (``moe_dtype: mxfp8``) instead of the reference's torchao swap.

Multi-GPU: launched by ``accelerate launch --config_file configs/fsdp_config.yaml`` Accelerate applies FSDP
itself; launched by ``torchrun`` the script asks the HF Trainer for ``full_shard auto_wrap`` over
``TransformerBlock`` (reference: train_production.py:518-529), taking prefetch / offload switches from
``--fsdp_config`` (an Accelerate-style YAML such as ``configs/fsdp_config.yaml``).  Without ``accelerate``
installed the same file selects this framework's own parameter-sharded plan (FULL_SHARD per block, AdamW on
the shards, optional host offload) on the native loop.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# names the reference's script defines at module level; the two Trainer subclasses need ``transformers`` and are
# built on first use
from kolmogorov_moe_architecture_b200.training.hf import (MoEModelWrapper, OnTheFlyDataCollator,  # noqa: E402,F401
                                                          load_and_prepare_dataset)
from kolmogorov_moe_architecture_b200.training.script_api import load_config  # noqa: E402,F401


def __getattr__(name):
    if name in ("MoETrainer", "TrueLossLoggingCallback"):
        from kolmogorov_moe_architecture_b200.training.hf import make_hf_classes
        trainer, callback = make_hf_classes()
        return trainer if name == "MoETrainer" else callback
    raise AttributeError(name)
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def fsdp_settings(path, env=None):
    """What an Accelerate-style FSDP file (``fsdp_config:`` block) asks for, in both vocabularies.

    Returns ``{"distributed", "accelerate_owns_fsdp", "cpu_offload", "hf_kwargs"}``: ``hf_kwargs`` are the
    ``TrainingArguments`` entries for a torchrun launch (empty when Accelerate applies FSDP itself or the job
    has one process); ``cpu_offload`` is what the native parameter-sharded plan takes from the file."""
    env = os.environ if env is None else env
    world = int(env.get("WORLD_SIZE", "1") or 1)
    fc = {}
    if path:
        import yaml
        with open(path) as f:
            fc = (yaml.safe_load(f) or {}).get("fsdp_config", {}) or {}
    offload = bool(fc.get("fsdp_offload_params", False))
    owns = str(env.get("ACCELERATE_USE_FSDP", "")).lower() in ("1", "true", "yes")
    # sharding strategy and wrap policy in the words of ``TrainingArguments.fsdp``
    strategy = {"FULL_SHARD": "full_shard", "SHARD_GRAD_OP": "shard_grad_op", "HYBRID_SHARD": "hybrid_shard",
                "NO_SHARD": "no_shard"}.get(str(fc.get("fsdp_sharding_strategy", "FULL_SHARD")).upper(), "full_shard")
    by_layer = str(fc.get("fsdp_auto_wrap_policy", "TRANSFORMER_BASED_WRAP")).upper() == "TRANSFORMER_BASED_WRAP"
    hf = {}
    if world > 1 and not owns:
        hf = {"fsdp": strategy + " auto_wrap" + (" offload" if offload else ""),
              "fsdp_config": {**({"transformer_layer_cls_to_wrap": ["TransformerBlock"]} if by_layer
                                 else {"min_num_params": int(fc.get("fsdp_min_num_params", 1e8))}),
                              "state_dict_type": str(fc.get("fsdp_state_dict_type", "SHARDED_STATE_DICT")),
                              "backward_prefetch": str(fc.get("fsdp_backward_prefetch", "BACKWARD_PRE")).lower(),
                              "forward_prefetch": bool(fc.get("fsdp_forward_prefetch", True)),
                              "use_orig_params": bool(fc.get("fsdp_use_orig_params", True)),
                              "cpu_ram_efficient_loading": bool(fc.get("fsdp_cpu_ram_efficient_loading", True)),
                              "sync_module_states": bool(fc.get("fsdp_sync_module_states", True)),
                              "limit_all_gathers": bool(fc.get("fsdp_limit_all_gathers", True))}}
    return {"distributed": world > 1, "accelerate_owns_fsdp": owns, "cpu_offload": offload, "hf_kwargs": hf,
            "sharding_strategy": strategy, "sharded_state_dict": "SHARDED" in str(fc.get("fsdp_state_dict_type",
                                                                                        "SHARDED_STATE_DICT")).upper()}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, required=True)
    ap.add_argument("--resume_from_checkpoint", type=str, default=None)
    ap.add_argument("--max_steps", type=int, default=None)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--output_dir", type=str, default=None)
    ap.add_argument("--fsdp_config", type=str, default=None,
                    help="Accelerate-style FSDP settings (e.g. configs/fsdp_config.yaml) for multi-process runs")
    a = ap.parse_args(argv)
    fs = fsdp_settings(a.fsdp_config)
    import importlib.util
    if importlib.util.find_spec("accelerate") is None:
        # HF Trainer cannot be constructed without `accelerate`; run the same recipe (hybrid optimizer,
        # cosine schedule with warm-up, checkpoint-N directories with the newest three kept) on the native loop.
        print("accelerate is not installed: running the HF recipe on the native training loop")
        from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
        if fs["distributed"]:
            print("multi-process run: FULL_SHARD per transformer block on this framework's parameter-sharded plan"
                  + (" with host offload" if fs["cpu_offload"] else ""))
        return run_training(RunSpec(config_path=a.config, steps=a.max_steps, strict_config=True,
                                    weights="bf16" if fs["distributed"] else "fp32_autocast",
                                    optimizer_family="hybrid", checkpoint_format="C",
                                    checkpoint_dir=a.output_dir, resume=a.resume_from_checkpoint,
                                    data_mode="synthetic" if a.synthetic else "streaming",
                                    shard_params=fs["distributed"], cpu_offload=fs["distributed"] and fs["cpu_offload"]))
    import torch
    from torch.utils.data import Dataset
    from transformers import TrainingArguments
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.training.hf import MoEModelWrapper, make_hf_classes
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_strict, section
    y = load_yaml(a.config)
    tc, oc, dc = section(y, "training"), section(y, "optimizer"), section(y, "data")
    mp = y.get("mixed_precision") or {}
    over = {"moe_dtype": "mxfp8"} if mp.get("fp8") else {}
    cfg = model_config_strict(y, **over)
    model = MoEModelWrapper(MoETransformer(cfg))
    MoETrainer, TrueLoss = make_hf_classes()

    class Rows(Dataset):
        def __init__(self, n, seed):
            g = torch.Generator().manual_seed(seed)
            self.x = torch.randint(1, cfg.vocab_size, (n, cfg.max_seq_len), generator=g)

        def __len__(self):
            return self.x.shape[0]

        def __getitem__(self, i):
            return {"input_ids": self.x[i], "labels": self.x[i]}

    if a.synthetic:
        train_ds, eval_ds = Rows(256, 0), Rows(16, 1)
    else:
        from kolmogorov_moe_architecture_b200.data import DolmaStreamingDataset, TokenizerWrapper
        tok = TokenizerWrapper(dc.get("tokenizer_name", "gpt2"))
        train_ds = DolmaStreamingDataset(tok, cfg.max_seq_len, cfg.n_pred_tokens, "train", True, cfg.vocab_size)
        eval_ds = None
    steps = a.max_steps or max(1, tc["total_tokens"] // (tc["batch_size"] * cfg.max_seq_len *
                                                          tc["gradient_accumulation_steps"]))
    cuda = torch.cuda.is_available()
    hfc, wb, evc = y.get("huggingface") or {}, y.get("wandb") or {}, y.get("evaluation") or {}
    report = ["wandb"] if (wb.get("enabled") or hfc.get("use_wandb")) else []
    if report:
        os.environ.setdefault("WANDB_PROJECT", str(wb.get("project", "moe-training")))
        if wb.get("entity"):
            os.environ.setdefault("WANDB_ENTITY", str(wb["entity"]))
    if hfc.get("logging_dir"):
        report.append("tensorboard")
    extra = {}
    if evc.get("enabled") and eval_ds is not None:
        # evaluation.eval_steps batches every evaluation.eval_interval steps (training.eval_interval as fallback)
        n_eval = int(evc.get("eval_steps", 100)) * tc["batch_size"]
        eval_ds = torch.utils.data.Subset(eval_ds, range(min(n_eval, len(eval_ds))))
        extra = {"eval_strategy": "steps", "eval_steps": int(evc.get("eval_interval", tc.get("eval_interval", 500)))}
    else:
        eval_ds = None
    args = TrainingArguments(
        output_dir=a.output_dir or tc["checkpoint_dir"], max_steps=steps,
        per_device_train_batch_size=tc["batch_size"], gradient_accumulation_steps=tc["gradient_accumulation_steps"],
        learning_rate=tc["max_lr"], warmup_steps=min(tc["warmup_steps"], max(steps - 1, 0)),
        max_grad_norm=tc["gradient_clip_norm"], logging_steps=tc["log_interval"], save_steps=tc["save_interval"],
        save_total_limit=int(hfc.get("save_total_limit", 3)), bf16=bool(mp.get("bf16", cuda)) and cuda,
        report_to=report, run_name=wb.get("run_name"), logging_dir=hfc.get("logging_dir"),
        seed=int(hfc.get("seed", 42)), remove_unused_columns=False,
        dataloader_num_workers=0, use_cpu=not cuda, **extra, **fs["hf_kwargs"])
    trainer = MoETrainer(oc, tc, tc["log_interval"], model=model, args=args, train_dataset=train_ds,
                         eval_dataset=eval_ds, callbacks=[TrueLoss(tc["gradient_accumulation_steps"])])
    try:
        trainer.train(resume_from_checkpoint=a.resume_from_checkpoint)
    except KeyboardInterrupt:
        print("interrupted: the newest checkpoint-N directory holds the last saved state")
    return trainer


if __name__ == "__main__":
    main()
