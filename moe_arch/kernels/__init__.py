from kolmogorov_moe_architecture_b200.kernels import *  # noqa: F401,F403
from kolmogorov_moe_architecture_b200.kernels import grouped_swiglu_forward, grouped_swiglu_with_grad, is_kernel_available  # noqa: F401
