"""``sparse`` and ``expert_parallel`` MoE implementations
(reference: moe_arch/model/sparse_moe.py:292-652).

The reference's expert-parallel layer exchanges tokens with plain c10d
``all_to_all_single`` calls, which autograd does not see, so its experts, router
and inputs receive no language-model gradient through the exchange
(sparse_moe.py:540-603).  Here dispatch and combine are differentiable
(:mod:`..parallel.ep`), and the expert parameters are marked so the data-parallel
sharder leaves them out of its shard group.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


class SparseGroupedExpertsPyTorch(nn.Module):
    """Stacked SwiGLU experts, truncated-normal init (std = 1/sqrt(3 fan_in), cut at 2 std)."""

    def __init__(self, n_experts: int, d_model: int, d_ff: int, activation: str = "swiglu",
                 moe_dtype: str = "bf16"):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff, self.moe_dtype = n_experts, d_model, d_ff, moe_dtype
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        for w in (self.w1, self.w2, self.w3):
            std = math.sqrt(1.0 / 3.0) / math.sqrt(w.shape[1])
            nn.init.trunc_normal_(w, mean=0.0, std=std, a=-2 * std, b=2 * std)

    def forward(self, x: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor,
                keep: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.grouped_swiglu(x, self.w1, self.w2, self.w3, expert_indices, expert_weights,
                                  keep, self.moe_dtype)


SparseGroupedExperts = SparseGroupedExpertsPyTorch


def get_sparse_experts(n_experts: int, d_model: int, d_ff: int, use_triton: bool = False, **kw) -> nn.Module:
    """Factory kept for API parity (sparse_moe.py:659-687); there is one implementation."""
    return SparseGroupedExpertsPyTorch(n_experts, d_model, d_ff, **kw)


class ExpertParallelMoE(nn.Module):
    """Experts block-partitioned over the ranks of ``process_group``.

    Router: a single ``Linear(d, E)``; top-k is taken on the *logits* and the weights
    are a softmax over those k logits (sparse_moe.py:456,490-493) - this differs from
    ``Router`` and is kept so checkpoints keyed ``expert_parallel_layer.*`` behave the
    same.  Aux loss: ``w_lb * E * sum_i c_i P_i + w_z * mean(lse^2)`` with c_i the mean
    number of slots per token routed to expert i (so it sums to top_k).
    """

    def __init__(self, config, layer_idx: int, process_group=None):
        super().__init__()
        import torch.distributed as dist
        if process_group is None and dist.is_available() and dist.is_initialized():
            from ..parallel.mesh import default_ep_group
            process_group = default_ep_group()
        self.config, self.layer_idx, self.process_group = config, layer_idx, process_group
        if dist.is_available() and dist.is_initialized():
            self.world_size = dist.get_world_size(process_group)
            self.rank = dist.get_rank(process_group)
        else:
            self.world_size, self.rank = 1, 0
        self.n_experts, self.top_k = config.n_experts, config.moe_top_k
        self.d_model, self.d_ff = config.d_model, config.d_ff_expert
        assert self.n_experts % self.world_size == 0, (
            f"n_experts ({self.n_experts}) must be divisible by world_size ({self.world_size})")
        self.n_local_experts = self.n_experts // self.world_size
        self.expert_start_idx = self.rank * self.n_local_experts
        self.expert_end_idx = self.expert_start_idx + self.n_local_experts
        self.router = Linear(config.d_model, config.n_experts, bias=False)
        self.local_experts = SparseGroupedExpertsPyTorch(
            self.n_local_experts, config.d_model, config.d_ff_expert,
            moe_dtype=getattr(config, "moe_dtype", "bf16"))
        for p in self.local_experts.parameters():
            p._kmoe_expert_parallel = True          # excluded from data-parallel sharding/averaging
        self.capacity_factor = config.moe_capacity_factor
        self.drop_tokens = getattr(config, "moe_drop_tokens", False)
        self.aux_loss = 0.0
        self.last_expert_counts = None
        # "auto": peer-pointer kernels when available, else all_to_all; "p2p" / "all_to_all" force one
        import os
        self.transport = os.environ.get("KMOE_EP_TRANSPORT", "auto")

    def _compute_aux_loss(self, logits: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        probs = F.softmax(logits, dim=-1)
        c = F.one_hot(idx, self.n_experts).float().sum(dim=1).mean(dim=0)
        lb = self.n_experts * (c * probs.mean(dim=0)).sum()
        z = torch.logsumexp(logits, dim=-1).pow(2).mean()
        return self.config.moe_load_balance_loss_weight * lb + self.config.moe_router_z_loss_weight * z

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, d = x.shape
        xf = x.reshape(-1, d)
        logits = self.router(xf)
        topv, idx = torch.topk(logits, self.top_k, dim=-1)
        w = F.softmax(topv, dim=-1)
        if self.training:
            self.aux_loss = self._compute_aux_loss(logits, idx)
        else:
            self.aux_loss = 0.0
        with torch.no_grad():
            self.last_expert_counts = torch.bincount(idx.reshape(-1), minlength=self.n_experts)
        keep = None
        if self.drop_tokens:
            cap = int(math.ceil(self.capacity_factor * idx.numel() / self.n_experts))
            keep = ops.capacity_keep_mask(idx, self.n_experts, cap)
        if self.world_size == 1:
            return self.local_experts(xf, idx, w, keep).reshape(B, S, d)
        le = self.local_experts
        if self.transport != "all_to_all" and le.moe_dtype in ("bf16", "mxfp8"):
            from ..parallel import ep_p2p
            if ep_p2p.fused_available(xf, le.w1, le.moe_dtype):
                # permute + exchange fused over NVLink peer pointers; no host read, no NCCL
                try:
                    out = ep_p2p.expert_parallel_ffn_fused(xf, idx, w, le.w1, le.w2, le.w3, self.n_experts,
                                                           self.process_group, keep=keep,
                                                           slot_cap=cap if keep is not None else None,
                                                           moe_dtype=le.moe_dtype)
                    return out.reshape(B, S, d)
                except ep_p2p.EPUnavailable as e:
                    if self.transport == "p2p":
                        raise
                    print(f"[kmoe] peer-pointer expert exchange unavailable ({e}); using all_to_all", flush=True)
                    self.transport = "all_to_all"
            if self.transport == "p2p":
                raise RuntimeError("expert-parallel transport 'p2p' needs CUDA bf16 tensors and peer access")
        from ..parallel.ep import expert_parallel_ffn
        out = expert_parallel_ffn(xf, idx, w, self.local_experts, self.n_experts,
                                  self.process_group, keep=keep)
        return out.reshape(B, S, d)


def benchmark_sparse_vs_batched(n_experts: int = 64, d_model: int = 2048, d_ff: int = 1536, n_tokens: int = 8192,
                                top_k: int = 2, n_iters: int = 20, device=None):
    """``SparseGroupedExpertsPyTorch`` against ``BatchedMoEOptimized`` with the same weights: agreement of the
    outputs and forward time (reference: moe_arch/model/sparse_moe.py:694-789, at d_ff 1524; 1536 here: the
    kernels take widths that are multiples of 64).  In this framework both names run the grouped kernel, so the
    figures also show that the two entry points cost the same."""
    import torch
    from ._bench import default_device, report, routed_inputs, time_ms
    from .triton_moe import BatchedMoEOptimized
    device = device or default_device()
    dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    x, idx, w = routed_inputs(n_tokens, d_model, n_experts, top_k, device, dtype)
    sparse = SparseGroupedExpertsPyTorch(n_experts, d_model, d_ff).to(device).to(dtype)
    batched = BatchedMoEOptimized(n_experts, d_model, d_ff).to(device).to(dtype)
    with torch.no_grad():
        for a, b in zip(batched.parameters(), sparse.parameters()):
            a.copy_(b)
        diff = float((sparse(x, idx, w).float() - batched(x, idx, w).float()).abs().max())
        times = {"batched": time_ms(lambda: batched(x, idx, w), device, iters=n_iters),
                 "sparse": time_ms(lambda: sparse(x, idx, w), device, iters=n_iters)}
    print(f"max |sparse - batched| = {diff:.6f}")
    times = report(f"{n_experts} experts, d_model {d_model}, d_ff {d_ff}, {n_tokens} tokens, top-{top_k}", times, "batched")
    times["max_diff"] = diff
    return times
