from kolmogorov_moe_architecture_b200.models.fused_moe import FusedSparseMoE, OptimizedGroupedExperts  # noqa: F401
from kolmogorov_moe_architecture_b200.models.fused_moe import benchmark_fused_vs_original  # noqa: F401
