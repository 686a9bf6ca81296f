"""Sparse distillation of dense transformers into mixture-of-experts layers (the reference's
``Experiments/sparse_distillation`` package; importable under that name as well)."""
from .convert import SparseModelWrapper, convert_to_sparse, replace_ffn_with_moe  # noqa: F401
from .distill import DistillationConfig, MoEDistillationLayer, SparseDistillationTrainer  # noqa: F401
from .hooks import FFNActivation, FFNActivationCache, StreamingFFNExtractor  # noqa: F401
