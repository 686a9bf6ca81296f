"""Benchmark variants kept for API parity with the reference's ``moe_arch/model/triton_moe.py``
(``TritonGroupedExperts``, ``TritonGroupedExpertsFused``, ``BatchedMoE``, ``BatchedMoEOptimized``,
``sort_tokens_by_expert``).  They are one implementation here - the grouped tcgen05 kernel -
so the names are aliases; no Triton is involved."""
from __future__ import annotations

import torch

from .moe import GroupedExperts


def sort_tokens_by_expert(expert_indices: torch.Tensor, n_experts: int):
    """Stable sort of the flat (token, slot) assignments by expert.
    Returns (sorted_token_idx, sorted_expert_ids, sort_order, seg_starts, seg_ends)."""
    T, k = expert_indices.shape
    flat = expert_indices.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = torch.arange(T, device=flat.device).repeat_interleave(k)[order]
    counts = torch.bincount(flat, minlength=n_experts)
    ends = torch.cumsum(counts, 0)
    return tok, flat[order], order, ends - counts, ends


class TritonGroupedExperts(GroupedExperts):
    pass


class TritonGroupedExpertsFused(GroupedExperts):
    pass


class BatchedMoE(GroupedExperts):
    pass


class BatchedMoEOptimized(GroupedExperts):
    pass
