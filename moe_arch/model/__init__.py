from kolmogorov_moe_architecture_b200.models import *  # noqa: F401,F403
