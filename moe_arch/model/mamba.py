from kolmogorov_moe_architecture_b200.models.mamba import Mamba, MambaBlock, MambaExpert, RoutingMamba, SimpleSSM  # noqa: F401
