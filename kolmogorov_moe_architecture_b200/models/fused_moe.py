"""``FusedSparseMoE`` and ``OptimizedGroupedExperts`` (API of the reference's
``moe_arch/model/fused_moe.py``).  In the reference "fused" is an aspiration - the router is
PyTorch and the experts a Python loop with a host sync per expert (fused_moe.py:249-253,300-319);
here both classes run the one grouped tcgen05 kernel path, keeping their parameter names
(``router_weight`` (d, E), ``w1/w2/w3``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops


def _init(w):
    nn.init.uniform_(w, -1.0 / math.sqrt(w.shape[1]), 1.0 / math.sqrt(w.shape[1]))


class OptimizedGroupedExperts(nn.Module):
    def __init__(self, n_experts: int, d_model: int, d_ff: int):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff = n_experts, d_model, d_ff
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        for w in (self.w1, self.w2, self.w3):
            _init(w)

    def forward(self, x, expert_indices, expert_weights):
        return ops.grouped_swiglu(x, self.w1, self.w2, self.w3, expert_indices, expert_weights)


class FusedSparseMoE(nn.Module):
    def __init__(self, d_model: int, d_ff: int, n_experts: int, top_k: int = 2):
        super().__init__()
        self.d_model, self.d_ff, self.n_experts, self.top_k = d_model, d_ff, n_experts, top_k
        self.router_weight = nn.Parameter(torch.empty(d_model, n_experts))
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        nn.init.normal_(self.router_weight, std=0.02)
        for w in (self.w1, self.w2, self.w3):
            _init(w)
        self.aux_loss = 0.0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = x.reshape(-1, self.d_model)
        logits = flat @ self.router_weight
        w, idx = ops.topk_softmax_route(logits, self.top_k)
        if self.training:
            self.aux_loss = ops.moe_aux_loss(logits, idx, self.n_experts, 0.01, 0.001)
        return ops.grouped_swiglu(flat, self.w1, self.w2, self.w3, idx, w).view(shape)


def benchmark_fused_vs_original(d_model: int = 512, d_ff: int = 1024, n_experts: int = 16, top_k: int = 2,
                                batch: int = 2, seq_len: int = 1024, n_iters: int = 20, device=None):
    """``FusedSparseMoE`` against ``MoELayer`` at the reference's shape (moe_arch/model/fused_moe.py:448-496):
    forward time of both on the same input."""
    from ..config import AdvancedMoEConfig
    from ._bench import default_device, report, time_ms
    from .moe import MoELayer
    device = device or default_device()
    dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    cfg = AdvancedMoEConfig(d_model=d_model, d_ff_expert=d_ff, n_experts=n_experts, moe_top_k=top_k, n_layers=4,
                            n_heads=max(d_model // 64, 1), n_kv_heads=max(d_model // 128, 1), head_dim=64,
                            moe_layers=(0,), mamba_enabled=False, mamba_layers=(), vocab_size=1000)
    original = MoELayer(cfg, layer_idx=0).to(device).to(dtype).eval()
    fused = FusedSparseMoE(d_model, d_ff, n_experts, top_k).to(device).to(dtype).eval()
    x = torch.randn(batch, seq_len, d_model, generator=torch.Generator().manual_seed(0)).to(device=device, dtype=dtype)
    with torch.no_grad():
        times = {"MoELayer": time_ms(lambda: original(x), device, iters=n_iters),
                 "FusedSparseMoE": time_ms(lambda: fused(x), device, iters=n_iters)}
    return report(f"{n_experts} experts, d_model {d_model}, d_ff {d_ff}, {batch} x {seq_len} tokens", times, "MoELayer")
