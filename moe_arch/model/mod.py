from kolmogorov_moe_architecture_b200.models.mod import MoDRouter  # noqa: F401
from kolmogorov_moe_architecture_b200.models.mod import MoDLayer  # noqa: F401
