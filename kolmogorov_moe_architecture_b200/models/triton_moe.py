"""Benchmark variants kept for API parity with the reference's ``moe_arch/model/triton_moe.py``
(``TritonGroupedExperts``, ``TritonGroupedExpertsFused``, ``BatchedMoE``, ``BatchedMoEOptimized``,
``sort_tokens_by_expert``).  They are one implementation here - the grouped tcgen05 kernel -
so the names are aliases; no Triton is involved."""
from __future__ import annotations

import torch

from .moe import GroupedExperts


def sort_tokens_by_expert(expert_indices: torch.Tensor, expert_weights=None, n_experts: int = None):
    """Stable sort of the flat (token, slot) assignments by expert (reference: triton_moe.py:160-198).

    ``sort_tokens_by_expert(expert_indices, expert_weights, n_experts)`` returns
    (sorted_token_indices, sorted_expert_ids, sorted_weights, segment_starts, segment_ends).
    Called without weights - ``sort_tokens_by_expert(expert_indices, n_experts)`` - the third result is the sort
    order itself (flat assignment index of every sorted position), from which any per-assignment tensor can be
    brought into the same order."""
    if n_experts is None and not torch.is_tensor(expert_weights):
        expert_weights, n_experts = None, expert_weights
    T, k = expert_indices.shape
    flat = expert_indices.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = torch.arange(T, device=flat.device).repeat_interleave(k)[order]
    counts = torch.bincount(flat, minlength=n_experts)
    ends = torch.cumsum(counts, 0)
    third = order if expert_weights is None else expert_weights.reshape(-1)[order]
    return tok, flat[order], third, ends - counts, ends


class TritonGroupedExperts(GroupedExperts):
    pass


class TritonGroupedExpertsFused(GroupedExperts):
    pass


class BatchedMoE(GroupedExperts):
    pass


class BatchedMoEOptimized(GroupedExperts):
    pass


def benchmark_moe_implementations(n_experts: int = 110, d_model: int = 2048, d_ff: int = 1024, n_tokens: int = 16384,
                                  top_k: int = 2, n_iters: int = 20, device=None):
    """Forward time of the four expert classes of this module on one routed batch, and their agreement (reference:
    moe_arch/model/triton_moe.py:709-799, where they are four different implementations; here they share the
    grouped kernel and differ in name only, which the equal times show)."""
    import torch
    from ._bench import default_device, report, routed_inputs, time_ms
    device = device or default_device()
    dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    x, idx, w = routed_inputs(n_tokens, d_model, n_experts, top_k, device, dtype)
    mods = {c.__name__: c(n_experts, d_model, d_ff).to(device).to(dtype)
            for c in (BatchedMoE, BatchedMoEOptimized, TritonGroupedExperts, TritonGroupedExpertsFused)}
    base = mods["BatchedMoE"]
    times, diffs = {}, {}
    with torch.no_grad():
        ref = base(x, idx, w).float()
        for name, m in mods.items():
            for a, b in zip(m.parameters(), base.parameters()):
                a.copy_(b)
            diffs[name] = float((m(x, idx, w).float() - ref).abs().max())
            times[name] = time_ms(lambda m=m: m(x, idx, w), device, iters=n_iters)
    print("max |difference| to BatchedMoE:", {k: round(v, 6) for k, v in diffs.items()})
    times = report(f"{n_experts} experts, d_model {d_model}, d_ff {d_ff}, {n_tokens} tokens, top-{top_k}", times, "BatchedMoE")
    times["max_diff"] = max(diffs.values())
    return times
