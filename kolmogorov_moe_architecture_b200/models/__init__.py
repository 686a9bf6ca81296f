from .attention import GroupedQueryAttention
from .embeddings import RMSNorm, RotaryPositionalEmbedding, TokenEmbedding, get_norm_layer
from .ffn import ExpertFFN, StandardFFN, SwiGLU, get_ffn_module
from .layers import TransformerBlock
from .mamba import Mamba, MambaBlock, MambaExpert, RoutingMamba, SimpleSSM
from .mod import MoDRouter
from .moe import ExpertChoiceRouter, GroupedExperts, GroupedExpertsExpertChoice, MoELayer, Router
from .sparse_moe import ExpertParallelMoE, SparseGroupedExperts, SparseGroupedExpertsPyTorch
from .transformer import MoETransformer
