"""Sharded data parallelism with whole-tensor ownership.

The reference shards everything FSDP-style (FULL_SHARD per ``TransformerBlock``: bf16
all-gather of every block's parameters in forward and again in backward, bf16
reduce-scatter of gradients; reference: train_distributed.py:275-319).  On a GPU with
180 GB of HBM the bf16 weights of the 5B model (11.7 GB) are cheap to replicate, so this
runtime keeps parameters replicated and shards only what is large and rank-private:
gradients after reduction and optimizer state.  Per step that is ONE reduce-scatter of the
flat gradient buffer and ONE all-gather of the updated parameters, instead of FSDP's two
all-gathers and one reduce-scatter per block.

Ownership is per tensor, not per flat byte range: every parameter (2-D matrices and 3-D
expert stacks included) belongs to exactly one rank, so Muon's Newton-Schulz runs on whole
matrices on the owner with no gather, and each rank orthogonalises only its share of the
matrices.  Rank r's tensors are packed into segment r of two flat buffers (parameters and
gradients) whose segments have equal size; ``reduce_scatter_tensor`` then hands each owner
the averaged gradients of exactly its tensors, and ``all_gather_into_tensor`` publishes the
updated tensors.  On CUDA with peer access the same two steps run as this library's own
kernels over NVLink peer pointers (:mod:`.p2p`), fused with the AdamW update.

Gradient accumulation needs no ``no_sync`` bookkeeping: gradients accumulate locally in the
flat buffer and are reduced once, when the step is taken.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..training.muon_optimizer import _EXCLUDE, HybridOptimizer, Muon
from ..training.optim_factory import make_adamw

_ALIGN = 128   # elements; keeps every tensor 256-byte aligned inside a segment


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def assign_owners(numels: List[int], world: int) -> List[int]:
    """Greedy balance by element count: largest tensor first onto the lightest rank.
    Deterministic, so every rank computes the same assignment."""
    load = [0] * world
    owner = [0] * len(numels)
    for i in sorted(range(len(numels)), key=lambda j: (-numels[j], j)):
        r = min(range(world), key=lambda q: (load[q], q))
        owner[i] = r
        load[r] += _round_up(numels[i], _ALIGN)
    return owner


class ShardedDataParallel:
    def __init__(self, model: torch.nn.Module, optimizer_kind: str = "muon", group=None,
                 lr: float = 1e-3, adamw_lr: float = 3e-4, momentum: float = 0.95,
                 weight_decay: float = 0.01, newton_iters: int = 5, use_p2p: Optional[bool] = None,
                 broadcast_from_rank0: bool = True, expert_params: bool = False, grad_scale: float = 1.0):
        """``expert_params=False``: all parameters except expert-parallel ones (``group`` = every
        data-parallel rank).  ``expert_params=True``: only the expert-parallel tensors, with
        ``group`` the ranks that hold replicas of the same experts and ``grad_scale = 1/ep``
        (an expert's gradient already sums the losses of the ep ranks that sent it tokens)."""
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        named: List[Tuple[str, torch.nn.Parameter]] = []
        seen = set()
        for n, p in model.named_parameters():
            if p.requires_grad and id(p) not in seen and \
                    bool(getattr(p, "_kmoe_expert_parallel", False)) == expert_params:
                seen.add(id(p))
                named.append((n, p))
        assert named, "no trainable parameters"
        self.named = named
        dtype, device = named[0][1].dtype, named[0][1].device
        assert all(p.dtype == dtype for _, p in named), "parameters must share one dtype"
        self.dtype, self.device = dtype, device
        owners = assign_owners([p.numel() for _, p in named], self.world)
        offsets = [0] * self.world
        self.slots: List[Tuple[int, int]] = []          # (owner, offset in segment)
        for (n, p), r in zip(named, owners):
            self.slots.append((r, offsets[r]))
            offsets[r] += _round_up(p.numel(), _ALIGN)
        self.seg = _round_up(max(offsets) if offsets else _ALIGN, _ALIGN)
        total = self.seg * self.world
        self.use_p2p = False
        if use_p2p is None:
            use_p2p = False
        self.flat_param, self.flat_grad, self.p2p = self._alloc(total, use_p2p)
        with torch.no_grad():
            for (n, p), (r, off) in zip(named, self.slots):
                view = self.flat_param[r * self.seg + off: r * self.seg + off + p.numel()].view_as(p)
                view.copy_(p.data)
                p.data = view
                p.grad = self.flat_grad[r * self.seg + off: r * self.seg + off + p.numel()].view_as(p)
        if broadcast_from_rank0 and self.world > 1:
            dist.broadcast(self.flat_param, src=dist.get_global_rank(group, 0) if group is not None else 0,
                           group=group)
        self.owned = [(n, p) for (n, p), (r, _) in zip(named, self.slots) if r == self.rank]
        self.optimizer = self._build_optimizer(optimizer_kind, lr, adamw_lr, momentum, weight_decay, newton_iters)
        self._sync = True
        self.grad_scale = grad_scale

    # ------------------------------------------------------------------ set-up
    def _alloc(self, total: int, use_p2p: bool):
        if use_p2p and self.device.type == "cuda" and self.world > 1:
            try:
                from .p2p import SymmetricBuffers
                sb = SymmetricBuffers(total, self.dtype, self.device, self.group)
                self.use_p2p = True
                return sb.param, sb.grad, sb
            except Exception as e:  # pragma: no cover - needs multi-GPU peer access
                if self.rank == 0:
                    print(f"[zero] symmetric memory unavailable ({e}); using NCCL collectives")
        fp = torch.zeros(total, dtype=self.dtype, device=self.device)
        fg = torch.zeros(total, dtype=self.dtype, device=self.device)
        return fp, fg, None

    def _build_optimizer(self, kind, lr, adamw_lr, momentum, wd, iters):
        if kind == "adamw":
            ps = [p for _, p in self.owned]
            return make_adamw(ps, adamw_lr, weight_decay=wd) if ps else None
        muon_p, adamw_p = [], []
        for n, p in self.owned:
            nl = n.lower()
            is_w = ".weight" in nl and not any(t in nl for t in _EXCLUDE)
            (muon_p if (is_w and p.dim() == 2) else adamw_p).append(p)
        muon = Muon(muon_p, lr=lr, momentum=momentum, weight_decay=wd, newton_iters=iters) if muon_p else None
        adamw = make_adamw(adamw_p, adamw_lr, weight_decay=wd) if adamw_p else None
        return HybridOptimizer(muon, adamw)

    # -------------------------------------------------------------------- step
    def set_sync(self, flag: bool) -> None:
        self._sync = flag

    def own_slice(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.rank * self.seg: (self.rank + 1) * self.seg]

    def _reduce_gradients(self) -> None:
        if self.world == 1:
            return
        if self.use_p2p:
            self.p2p.reduce_scatter_mean(self.rank, self.seg)
            return
        backend = dist.get_backend(self.group)
        if backend == "nccl":
            dist.reduce_scatter_tensor(self.own_slice(self.flat_grad), self.flat_grad, op=dist.ReduceOp.AVG,
                                       group=self.group)
        else:
            dist.all_reduce(self.flat_grad, group=self.group)
            self.flat_grad.div_(self.world)

    def _publish_parameters(self) -> None:
        if self.world == 1:
            return
        if self.use_p2p:
            self.p2p.all_gather_params(self.rank, self.seg)
            return
        dist.all_gather_into_tensor(self.flat_param, self.own_slice(self.flat_param).clone()
                                    if dist.get_backend(self.group) != "nccl" else self.own_slice(self.flat_param),
                                    group=self.group)

    def reduce(self) -> None:
        self._reduce_gradients()
        if self.grad_scale != 1.0:
            self.own_slice(self.flat_grad).mul_(self.grad_scale)

    def owned_sq_norm(self) -> torch.Tensor:
        return self.own_slice(self.flat_grad).float().pow(2).sum()

    def scale_owned(self, coef: torch.Tensor) -> None:
        g = self.own_slice(self.flat_grad)
        g.mul_(coef.to(g.dtype))

    def finish(self, optimizer=None) -> None:
        opt = optimizer if optimizer is not None else self.optimizer
        if opt is not None:
            opt.step()
        self._publish_parameters()
        self.flat_grad.zero_()

    def reduce_clip_and_step(self, optimizer=None, max_norm: Optional[float] = 1.0) -> torch.Tensor:
        """Reduce gradients to their owners, clip by the global norm, update the owned
        tensors, publish them, and clear the gradient buffer.  Returns the global gradient
        norm (device tensor)."""
        return ParallelPlan([self]).reduce_clip_and_step(optimizer, max_norm)

    # ------------------------------------------------------------- checkpoints
    def owned_names(self) -> List[str]:
        return [n for n, _ in self.owned]

    def optimizer_state_dict(self) -> Dict:
        """State of this rank's shard plus the names it covers (for sharded checkpoints)."""
        return {"rank": self.rank, "world": self.world, "owned": self.owned_names(),
                "state": self.optimizer.state_dict() if self.optimizer is not None else None}

    def load_optimizer_state_dict(self, sd: Dict) -> None:
        assert sd["owned"] == self.owned_names(), "optimizer shard does not match this rank's ownership"
        if self.optimizer is not None and sd["state"] is not None:
            self.optimizer.load_state_dict(sd["state"])


class ParallelPlan:
    """One or more parameter pools (dense parameters over all ranks; expert-parallel
    parameters over their replica group) stepped together with a single global-norm clip."""

    def __init__(self, pools: List[ShardedDataParallel], norm_group=None):
        self.pools, self.norm_group = pools, norm_group
        self.optimizer = pools[0].optimizer

    def set_sync(self, flag: bool) -> None:
        for p in self.pools:
            p.set_sync(flag)

    def reduce_clip_and_step(self, optimizer=None, max_norm: Optional[float] = 1.0) -> torch.Tensor:
        for p in self.pools:
            p.reduce()
        sq = sum(p.owned_sq_norm() for p in self.pools)
        if dist.is_initialized() and dist.get_world_size(self.norm_group) > 1:
            dist.all_reduce(sq, group=self.norm_group)
        total = sq.sqrt()
        if max_norm is not None and max_norm > 0:
            coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
            for p in self.pools:
                p.scale_owned(coef)
        for i, p in enumerate(self.pools):
            p.finish(optimizer if (optimizer is not None and i == 0 and len(self.pools) == 1) else None)
        return total

    @property
    def param_groups(self):
        out = []
        for p in self.pools:
            if p.optimizer is not None:
                out.extend(p.optimizer.param_groups)
        return out
