from kolmogorov_moe_architecture_b200.models.ffn import ExpertFFN, StandardFFN, SwiGLU, get_ffn_module  # noqa: F401
