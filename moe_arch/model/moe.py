from kolmogorov_moe_architecture_b200.models.moe import ExpertChoiceRouter, GroupedExperts, GroupedExpertsExpertChoice, MoELayer, Router  # noqa: F401
from kolmogorov_moe_architecture_b200.models.moe import Expert  # noqa: F401
