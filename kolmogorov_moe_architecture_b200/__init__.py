"""B200-native hybrid-MoE training framework.

Public API mirrors the reference package ``moe_arch``: ``AdvancedMoEConfig``,
``MoETransformer``, the config presets, the training library (losses, Muon
optimizers, schedulers, ``Trainer``) and the data helpers.
"""
from .config import (AdvancedMoEConfig, get_3b_config, get_5b_config, get_bench_5b_config,
                     get_test_config, get_tiny_debug_config)
from .models.transformer import MoETransformer

__version__ = "0.1.0"
__all__ = ["AdvancedMoEConfig", "MoETransformer", "get_5b_config", "get_3b_config",
           "get_test_config", "get_bench_5b_config", "get_tiny_debug_config"]
