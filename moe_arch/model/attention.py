from kolmogorov_moe_architecture_b200.models.attention import GroupedQueryAttention  # noqa: F401
