from kolmogorov_moe_architecture_b200.config import *  # noqa: F401,F403
from kolmogorov_moe_architecture_b200.config import AdvancedMoEConfig, get_3b_config, get_5b_config, get_test_config  # noqa: F401
