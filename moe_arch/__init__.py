"""Import-path compatibility: ``moe_arch.*`` resolves to ``kolmogorov_moe_architecture_b200``."""
from kolmogorov_moe_architecture_b200 import *  # noqa: F401,F403
from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer  # noqa: F401
