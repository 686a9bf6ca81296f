"""YAML configuration loading.

One schema for every entrypoint: sections ``model`` (fields of ``AdvancedMoEConfig``),
``training``, ``optimizer``, ``data``, ``mixed_precision``, ``wandb``, ``evaluation``,
``huggingface`` (reference: configs/production_training.yaml, configs/training_4.5b.yaml).

Two ways to build the model config, mirroring the reference's two families of loaders:
* ``model_config_strict``   - ``AdvancedMoEConfig(**yaml['model'])``; unknown keys raise
  (scripts/train.py:103, train_production.py:369, train_custom.py:979).
* ``model_config_tolerant`` - field-by-field with the fallback values used by the single-GPU
  and distributed scripts when a key is missing (train.py:473-504): no MoE / Mamba layers,
  one prediction head, dropout forced to 0.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import yaml

from ..config import AdvancedMoEConfig

SECTIONS = ("model", "training", "optimizer", "data", "mixed_precision", "wandb", "evaluation", "huggingface")

TRAINING_DEFAULTS = dict(total_tokens=1_000_000_000, batch_size=8, gradient_accumulation_steps=1, max_lr=3e-4,
                         min_lr_ratio=0.1, warmup_steps=2000, gradient_clip_norm=1.0, weight_decay=0.01,
                         checkpoint_dir="./checkpoints", save_interval=1000, log_interval=10, eval_interval=1000,
                         resume_from=None)
OPTIMIZER_DEFAULTS = dict(type="adamw", adamw_lr=3e-4, adamw_betas=[0.9, 0.95], muon_lr=0.02, momentum=0.95,
                          nesterov=True, weight_decay=0.01, backend="newton", newton_iters=5, norm_lr=None)
DATA_DEFAULTS = dict(dataset_name=None, dataset_config=None, tokenizer_name="gpt2", max_examples=None,
                     use_streaming=True, tokenize_on_fly=True, num_workers=0, use_document_attention_mask=False,
                     use_memory_mapped=False, data_path=None)


def load_yaml(path: str) -> Dict[str, Any]:
    with open(path, "r") as f:
        cfg = yaml.safe_load(f) or {}
    unknown = [k for k in cfg if k not in SECTIONS]
    if unknown:
        raise KeyError(f"{path}: unknown top-level section(s) {unknown}; expected {SECTIONS}")
    return cfg


def section(cfg: Dict[str, Any], name: str) -> Dict[str, Any]:
    base = {"training": TRAINING_DEFAULTS, "optimizer": OPTIMIZER_DEFAULTS, "data": DATA_DEFAULTS}.get(name, {})
    out = dict(base)
    out.update(cfg.get(name) or {})
    return out


def model_config_strict(cfg: Dict[str, Any], **overrides) -> AdvancedMoEConfig:
    m = dict(cfg.get("model") or {})
    m.update(overrides)
    return AdvancedMoEConfig(**m)


def model_config_tolerant(cfg: Dict[str, Any], seq_len: Optional[int] = None, **overrides) -> AdvancedMoEConfig:
    m = cfg.get("model") or {}
    g = m.get
    kw = dict(
        vocab_size=g("vocab_size", 50000), d_model=g("d_model", 2048), n_layers=g("n_layers", 32),
        n_heads=g("n_heads", 16), n_kv_heads=g("n_kv_heads", 4), head_dim=g("head_dim", 128),
        d_ff=g("d_ff", 5632), d_ff_expert=g("d_ff_expert", 2816),
        max_seq_len=seq_len if seq_len is not None else g("max_seq_len", 2048),
        n_experts=g("n_experts", 16), moe_top_k=g("moe_top_k", 2),
        moe_capacity_factor=g("moe_capacity_factor", 1.25),
        moe_load_balance_loss_weight=g("moe_load_balance_loss_weight", 0.01),
        moe_router_z_loss_weight=g("moe_router_z_loss_weight", 0.001),
        moe_layers=tuple(g("moe_layers", [])), moe_implementation=g("moe_implementation", "batched"),
        moe_routing=g("moe_routing", "token_choice"), moe_balanced_routing=g("moe_balanced_routing", False),
        mod_enabled=g("mod_enabled", True), mod_capacity_factor=g("mod_capacity_factor", 0.75),
        mod_router_hidden_dim=g("mod_router_hidden_dim", 128),
        mod_load_balance_loss_weight=g("mod_load_balance_loss_weight", 0.001),
        mamba_enabled=g("mamba_enabled", False), mamba_layers=tuple(g("mamba_layers", [])),
        n_pred_tokens=g("n_pred_tokens", 1), aux_loss_weights=tuple(g("aux_loss_weights", [1.0])),
        use_flash_attention=g("use_flash_attention", True),
        dropout=0.0, attention_dropout=0.0, residual_dropout=0.0)
    for k in ("ssm_state_dim", "ssm_expansion", "rope_theta", "norm_type", "norm_eps", "ffn_activation",
              "tie_word_embeddings", "init_std", "mamba_moe_mode", "moe_dtype", "ep_size", "moe_drop_tokens",
              "mamba_impl"):
        if k in m:
            kw[k] = m[k]
    kw.update(overrides)
    return AdvancedMoEConfig(**kw)
