from kolmogorov_moe_architecture_b200.models.embeddings import *  # noqa: F401,F403
from kolmogorov_moe_architecture_b200.models.embeddings import RMSNorm, RotaryPositionalEmbedding, TokenEmbedding, get_norm_layer  # noqa: F401
