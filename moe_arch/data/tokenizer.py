from kolmogorov_moe_architecture_b200.data.tokenizer import TokenizerWrapper  # noqa: F401
