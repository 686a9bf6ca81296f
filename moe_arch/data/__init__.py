from kolmogorov_moe_architecture_b200.data import *  # noqa: F401,F403
