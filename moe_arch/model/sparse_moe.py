from kolmogorov_moe_architecture_b200.models.sparse_moe import ExpertParallelMoE, SparseGroupedExperts, SparseGroupedExpertsPyTorch, get_sparse_experts  # noqa: F401
from kolmogorov_moe_architecture_b200.models.sparse_moe import benchmark_sparse_vs_batched  # noqa: F401
