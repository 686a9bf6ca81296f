"""Expert parallelism: differentiable token dispatch / combine.

Experts are block-partitioned over the ranks of the expert-parallel group (rank r holds
experts [r * E/ws, (r+1) * E/ws)).  A forward does

    sort assignments by destination rank -> exchange rows -> local grouped SwiGLU
    -> exchange results back -> weighted sum into the tokens

Both exchanges are autograd functions whose backward is the reverse exchange, so the
language-model gradient reaches the experts, the router and the layer input - the
reference's exchange is built from raw ``all_to_all_single`` calls that autograd does not
see (reference: moe_arch/model/sparse_moe.py:540-603).  The routing weight is applied on
the source rank after the combine (mathematically the same as the reference, which applies
it on the expert rank, and it keeps d(loss)/d(weight) local).

Two transports:
* ``all_to_all_single`` with per-rank split sizes (NCCL on GPUs, gloo in CPU tests).  The
  split sizes have to be known on the host, which costs one device-to-host read per layer.
* On CUDA ranks with peer access, :mod:`.p2p` moves the rows with this library's own kernels
  that store straight into the destination rank's receive buffer over NVLink; capacities
  are static, counts stay on the device and nothing synchronises with the host.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    """Row exchange with variable split sizes; backward is the exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, in_splits: List[int], out_splits: List[int], group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        gi = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(gi, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return gi, None, None, None


def all_to_all_rows(x, in_splits, out_splits, group=None):
    return _AllToAll.apply(x, in_splits, out_splits, group)


def expert_parallel_ffn(x: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor, local_experts,
                        n_experts: int, group=None, keep: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x (T, d); idx, weights (T, k) with global expert ids; ``local_experts(x, ids, w, keep)``
    evaluates this rank's experts.  Returns (T, d)."""
    from ..ops import checks
    if checks.enabled():
        checks.index_range(idx, n_experts, "expert index")
        checks.routing_weights(weights)
        checks.keep_mask(keep, idx)
    ws = dist.get_world_size(group)
    T, d = x.shape
    k = idx.shape[1]
    n_local = n_experts // ws
    flat_e = idx.reshape(-1)
    tok = torch.arange(T, device=x.device).repeat_interleave(k)
    valid = torch.ones_like(flat_e, dtype=torch.bool) if keep is None else keep.reshape(-1)
    dest = torch.where(valid, flat_e // n_local, torch.full_like(flat_e, ws))   # dropped -> sentinel
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=ws + 1)[:ws]
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    in_splits = send_counts.tolist()            # the one host read of this transport
    out_splits = recv_counts.tolist()
    n_send = sum(in_splits)
    order = order[:n_send]
    x_send = x[tok[order]]
    lid_send = (flat_e[order] % n_local).contiguous()
    x_recv = all_to_all_rows(x_send, in_splits, out_splits, group)
    lid_recv = lid_send.new_empty(sum(out_splits))
    dist.all_to_all_single(lid_recv, lid_send, out_splits, in_splits, group=group)
    ones = torch.ones(x_recv.shape[0], 1, dtype=weights.dtype, device=x.device)
    y_recv = local_experts(x_recv, lid_recv.view(-1, 1), ones, None)
    y_back = all_to_all_rows(y_recv, out_splits, in_splits, group)
    w_sel = weights.reshape(-1)[order].unsqueeze(1).to(y_back.dtype)
    out = torch.zeros_like(x)
    return out.index_add(0, tok[order], y_back * w_sel)
