from kolmogorov_moe_architecture_b200.models.triton_moe import BatchedMoE, BatchedMoEOptimized, TritonGroupedExperts, TritonGroupedExpertsFused, sort_tokens_by_expert  # noqa: F401
from kolmogorov_moe_architecture_b200.models.triton_moe import benchmark_moe_implementations  # noqa: F401
