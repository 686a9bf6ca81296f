"""Import path of the reference (``Experiments.sparse_distillation``); the code lives in ``experiments/``."""
