from kolmogorov_moe_architecture_b200.training.lr_schedule import CosineScheduleWithWarmup, get_lr_scheduler  # noqa: F401
