"""Model configuration.

``AdvancedMoEConfig`` keeps every field, default and preset of the reference
dataclass (reference: moe_arch/model/config.py:12-353) so that YAML files and
checkpoints written for the reference load unchanged.  Three runtime knobs are
added; each defaults to the reference behaviour:

* ``mamba_moe_mode``  - what a layer listed in both ``moe_layers`` and
  ``mamba_layers`` becomes.  ``"routing_mamba"`` (default) is the reference
  behaviour (RoutingMamba + dense FFN, moe_arch/model/layers.py:58-82);
  ``"moe_ffn"`` builds a plain Mamba mixer followed by an MoE FFN.
* ``moe_dtype``       - ``"bf16"`` or ``"mxfp8"`` for the expert GEMMs.
* ``ep_size``         - expert-parallel degree (1 = experts replicated/sharded
  with the rest of the model).
* ``moe_drop_tokens`` - token-choice capacity with drops (off by default; the
  reference never drops for token choice, moe_arch/model/moe.py:213-294).
* ``mamba_impl``      - ``"mamba"`` (selective-scan block with the parameter
  names of the mamba_ssm package) or ``"simple"`` (the gated depthwise-conv
  fallback the reference builds when mamba_ssm is missing, mamba.py:54-86).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Optional, Tuple


def _default_moe_layers() -> Tuple[int, ...]:
    return tuple(i for i in range(32) if (i % 4 == 2) or (i % 4 == 3) or (i in (9, 17, 25)))


def _default_mamba_layers() -> Tuple[int, ...]:
    return tuple(i for i in range(32) if (i % 4 == 1) and i >= 5)


@dataclass
class AdvancedMoEConfig:
    # model size
    vocab_size: int = 50000
    d_model: int = 2048
    n_layers: int = 32
    max_seq_len: int = 2048
    # attention
    n_heads: int = 16
    n_kv_heads: int = 4
    head_dim: int = 128
    # FFN
    d_ff: int = 5632
    d_ff_expert: int = 2816
    ffn_activation: str = "swiglu"
    # MoE
    n_experts: int = 16
    moe_top_k: int = 2
    moe_capacity_factor: float = 1.25
    moe_load_balance_loss_weight: float = 0.01
    moe_router_z_loss_weight: float = 0.001
    moe_implementation: str = "batched"       # batched | sparse | expert_parallel
    moe_routing: str = "token_choice"         # token_choice | expert_choice
    moe_balanced_routing: bool = False
    moe_layers: Tuple[int, ...] = field(default_factory=_default_moe_layers)
    # Mixture of Depths
    mod_enabled: bool = True
    mod_capacity_factor: float = 0.75
    mod_load_balance_loss_weight: float = 0.001
    mod_router_hidden_dim: int = 128
    # Mamba
    mamba_enabled: bool = True
    ssm_state_dim: int = 16
    ssm_expansion: int = 2
    mamba_layers: Tuple[int, ...] = field(default_factory=_default_mamba_layers)
    # multi-token prediction
    n_pred_tokens: int = 4
    aux_loss_weights: Tuple[float, ...] = (1.0, 0.5, 0.3, 0.2)
    # positions
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    # regularisation
    dropout: float = 0.1
    attention_dropout: float = 0.1
    residual_dropout: float = 0.1
    # norm
    norm_type: str = "rmsnorm"
    norm_eps: float = 1e-5
    init_std: float = 0.02
    # training
    use_gradient_checkpointing: bool = True
    gradient_checkpointing_segments: int = 4
    use_flash_attention: bool = True
    tie_word_embeddings: bool = True
    device: str = "cuda"
    dtype: str = "bfloat16"
    # ---- additions (defaults reproduce the reference) ----
    mamba_moe_mode: str = "routing_mamba"     # routing_mamba | moe_ffn
    moe_dtype: str = "bf16"                   # bf16 | mxfp8
    ep_size: int = 1
    moe_drop_tokens: bool = False
    mamba_impl: str = "mamba"                 # mamba | simple

    def __post_init__(self):
        self.moe_layers = tuple(self.moe_layers)
        self.mamba_layers = tuple(self.mamba_layers)
        self.aux_loss_weights = tuple(self.aux_loss_weights)
        assert self.d_model % self.n_heads == 0, (
            f"d_model ({self.d_model}) must be divisible by n_heads ({self.n_heads})")
        assert self.n_heads % self.n_kv_heads == 0, (
            f"n_heads ({self.n_heads}) must be divisible by n_kv_heads ({self.n_kv_heads})")
        self.n_groups = self.n_heads // self.n_kv_heads
        assert all(0 <= i < self.n_layers for i in self.moe_layers), \
            "MoE layer indices must be within [0, n_layers)"
        assert all(0 <= i < self.n_layers for i in self.mamba_layers), \
            "Mamba layer indices must be within [0, n_layers)"
        assert len(self.aux_loss_weights) == self.n_pred_tokens, (
            f"aux_loss_weights length ({len(self.aux_loss_weights)}) must match "
            f"n_pred_tokens ({self.n_pred_tokens})")
        assert 0.0 < self.mod_capacity_factor <= 1.0, "mod_capacity_factor must be in (0, 1]"
        assert self.mamba_moe_mode in ("routing_mamba", "moe_ffn")
        assert self.moe_dtype in ("bf16", "mxfp8")
        assert self.mamba_impl in ("mamba", "simple")
        assert self.moe_implementation in ("batched", "sparse", "expert_parallel")
        assert self.moe_routing in ("token_choice", "expert_choice")
        assert self.ep_size >= 1 and self.n_experts % self.ep_size == 0, \
            "n_experts must be divisible by ep_size"

    # ------------------------------------------------------------------ layout
    def get_layer_type(self, layer_idx: int) -> Tuple[str, bool]:
        """(sequence mixer kind, listed in moe_layers) for a layer (config.py:144-155)."""
        kind = "mamba" if layer_idx in self.mamba_layers else "attention"
        return kind, layer_idx in self.moe_layers

    def layer_plan(self, layer_idx: int) -> Tuple[str, str]:
        """Resolved (mixer, ffn) kinds: mixer in {attention, mamba, routing_mamba},
        ffn in {dense, moe}."""
        is_mamba = self.mamba_enabled and layer_idx in self.mamba_layers
        is_moe = layer_idx in self.moe_layers
        if is_mamba and is_moe:
            if self.mamba_moe_mode == "routing_mamba":
                return "routing_mamba", "dense"
            return "mamba", "moe"
        if is_mamba:
            return "mamba", "dense"
        return "attention", ("moe" if is_moe else "dense")

    # -------------------------------------------------------------- parameters
    def count_parameters(self) -> dict:
        """Analytic estimate with the reference's formulas (config.py:157-261),
        including its fixed 15 M-per-Mamba-layer figure."""
        token_embed = self.vocab_size * self.d_model
        attn = (self.d_model * self.n_heads * self.head_dim
                + 2 * self.d_model * self.n_kv_heads * self.head_dim
                + self.n_heads * self.head_dim * self.d_model)
        ffn = 3 * self.d_model * self.d_ff
        moe_ffn = self.n_experts * 3 * self.d_model * self.d_ff_expert
        moe_router = self.d_model * 128 + 128 * self.n_experts
        mamba = 15_000_000
        mod_router = self.d_model * self.mod_router_hidden_dim + self.mod_router_hidden_dim
        L = range(self.n_layers)
        n_std_attn = sum(1 for i in L if i not in self.mamba_layers and i not in self.moe_layers)
        n_moe_attn = sum(1 for i in L if i not in self.mamba_layers and i in self.moe_layers)
        n_mamba_std = sum(1 for i in L if i in self.mamba_layers and i not in self.moe_layers)
        n_mamba_moe = sum(1 for i in L if i in self.mamba_layers and i in self.moe_layers)
        total_attn = (n_std_attn + n_moe_attn) * attn
        total_mamba = (n_mamba_std + n_mamba_moe) * mamba
        total_ffn = (n_std_attn + n_mamba_std) * ffn
        total_moe = (n_moe_attn + n_mamba_moe) * (moe_ffn + moe_router)
        total_mod = self.n_layers * mod_router if self.mod_enabled else 0
        total_norm = self.n_layers * 2 * self.d_model
        mt_heads = (self.n_pred_tokens - 1) * self.vocab_size * self.d_model
        lm_head = self.vocab_size * self.d_model
        total = (token_embed + total_attn + total_mamba + total_ffn + total_moe
                 + total_mod + total_norm + mt_heads + lm_head)
        return {
            "token_embeddings": token_embed, "attention": total_attn, "mamba": total_mamba,
            "standard_ffn": total_ffn, "moe_ffn": total_moe, "mod_routers": total_mod,
            "layer_norms": total_norm, "multi_token_heads": mt_heads, "lm_head": lm_head,
            "total": total, "total_billions": total / 1e9,
            "n_standard_attn_layers": n_std_attn, "n_moe_attn_layers": n_moe_attn,
            "n_mamba_standard_layers": n_mamba_std, "n_mamba_moe_layers": n_mamba_moe,
        }

    def to_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if not k.startswith("_")}

    @classmethod
    def from_dict(cls, config_dict: dict) -> "AdvancedMoEConfig":
        """Strict loader: unknown keys raise (``n_groups`` is derived and dropped)."""
        d = dict(config_dict)
        d.pop("n_groups", None)
        return cls(**d)

    @classmethod
    def from_dict_tolerant(cls, config_dict: dict) -> "AdvancedMoEConfig":
        """Tolerant loader: keeps known keys, ignores the rest, like the
        field-by-field ``.get()`` loaders of the reference's train.py:473-504."""
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in config_dict.items() if k in known})


def get_5b_config() -> AdvancedMoEConfig:
    return AdvancedMoEConfig()


def get_3b_config() -> AdvancedMoEConfig:
    """24-layer, 64-expert preset (reference config.py:280-333)."""
    moe_layers = tuple(i for i in range(24) if (i % 4 == 2) or (i % 4 == 3) or (i in (9, 17, 21)))
    mamba_layers = tuple(i for i in range(24) if (i % 4 == 1) and i >= 5)
    return AdvancedMoEConfig(
        d_model=1792, n_layers=24, n_heads=14, n_kv_heads=2, head_dim=128,
        d_ff=4928, d_ff_expert=2464, n_experts=64, moe_top_k=2,
        mod_capacity_factor=0.5, moe_layers=moe_layers, mamba_layers=mamba_layers)


def get_test_config() -> AdvancedMoEConfig:
    return AdvancedMoEConfig(
        vocab_size=1000, d_model=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=64,
        d_ff=704, d_ff_expert=352, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,),
        max_seq_len=128, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5))


def get_bench_5b_config(**overrides) -> AdvancedMoEConfig:
    """The 5B hybrid used by the headline benchmark: 32 layers as 8x the pattern
    [Attn+dense, Mamba+MoE, Attn+MoE, Attn+dense], vocab 50304."""
    kw = dict(
        vocab_size=50304,
        moe_layers=tuple(i for i in range(32) if i % 4 in (1, 2)),
        mamba_layers=tuple(i for i in range(32) if i % 4 == 1),
        mamba_moe_mode="moe_ffn", dropout=0.0, attention_dropout=0.0, residual_dropout=0.0)
    kw.update(overrides)
    return AdvancedMoEConfig(**kw)


def get_tiny_debug_config(**overrides) -> AdvancedMoEConfig:
    """4-layer CPU debug model: one pass of the repeating pattern, d=256."""
    kw = dict(
        vocab_size=50304, d_model=256, n_layers=4, n_heads=4, n_kv_heads=1, head_dim=64,
        d_ff=1024, d_ff_expert=1024, n_experts=4, moe_top_k=2, moe_layers=(1, 2),
        mamba_layers=(1,), max_seq_len=128, n_pred_tokens=4, mod_capacity_factor=0.75,
        dtype="float32", device="cpu", dropout=0.0, attention_dropout=0.0, residual_dropout=0.0)
    kw.update(overrides)
    return AdvancedMoEConfig(**kw)
