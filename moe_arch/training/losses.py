from kolmogorov_moe_architecture_b200.training.losses import MultiTokenPredictionLoss  # noqa: F401
