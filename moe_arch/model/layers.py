from kolmogorov_moe_architecture_b200.models.layers import TransformerBlock  # noqa: F401
