from kolmogorov_moe_architecture_b200.models.fp8_moe import FP8GroupedExperts, FP8Linear, FP8MoELayer, is_fp8_available  # noqa: F401
from kolmogorov_moe_architecture_b200.models.fp8_moe import benchmark_fp8_vs_bf16  # noqa: F401
