"""``Experiments.sparse_distillation`` and its submodules are the modules of ``experiments.sparse_distillation``."""
import importlib
import sys

_pkg = importlib.import_module("experiments.sparse_distillation")
for _name in ("convert", "data", "distill", "dynamic_experts", "example_usage", "finetune_eval", "generate_config", "hooks"):
    _mod = importlib.import_module(f"experiments.sparse_distillation.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod
from experiments.sparse_distillation import *  # noqa: E402,F401,F403
from experiments.sparse_distillation import (DistillationConfig, FFNActivationCache,  # noqa: E402,F401
                                             SparseDistillationTrainer)
