from kolmogorov_moe_architecture_b200.training.trainer import Trainer  # noqa: F401
