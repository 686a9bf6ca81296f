from kolmogorov_moe_architecture_b200.models.transformer import MoETransformer  # noqa: F401
